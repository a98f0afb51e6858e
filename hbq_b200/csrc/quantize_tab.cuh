// Interface between the table plans (quantize_lut.cu) and the byte-table HBQ kernels (quantize_tab.cu).
#pragma once
#include "quantize_dev.cuh"

namespace hbq {

// Byte form of one format's candidate table (see byte_table_build in quantize_lut.cu).
struct TabTable {
    int slot;                 // index of the format among the cached plans
    const uint32_t* host;     // `entries` 32-bit entries, host memory, valid for the life of the process
    int entries;              // a multiple of 4
    int base, hi;             // |a| patterns covered: entry e <-> pattern base + e, e <= hi - base
    uint16_t big_l1;          // smallest block scale whose product with the largest candidate value overflows fp16
    uint16_t rm[8];           // fp16(1 / m) for the eight E5M3 mantissas
};
bool hbq_tab_table(int mb, const float* tab, int nc, TabTable* out);

// Runs the byte-table kernel if the (validated) HBQ arguments fit it; *launched tells whether it did.
int hbq_tab_try_launch(const QArgs& qa, int mb, cudaStream_t stream, bool* launched);

}  // namespace hbq
