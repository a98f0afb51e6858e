"""Llama-architecture decoder with the reference's quantisation points, tensor- and sequence-parallel.

The reference patches Hugging Face's ``LlamaAttention`` / ``LlamaMLP`` with quantizer-carrying subclasses
(``QLlamaAttention.forward`` src/module.py:120-199, ``manual_sdpa`` :93-117, ``QLlamaMLP.forward`` :547-569) and
lets ``PTQ`` inject the quantizers (``q_attn`` src/ptq.py:259-290, ``q_mlp`` :309-324), quantise the weights once
(:360-382) and set the accumulation operator (:384-404).  This module restates that block -- RMSNorm, q/k/v
projections, rotary embedding, post-RoPE Q / K / V quantisation, scores, softmax with the probability quantizer,
``P @ V``, o_proj, RMSNorm, gate / up, SiLU * up, down -- on the library's kernels, with the quantizers attached by
``PTQConfig.q_attn`` / ``q_mlp`` exactly as the reference's ``PTQ`` attaches them.  The surrounding model
(embedding, residual stream, final norm, lm_head) follows ``transformers``' ``LlamaForCausalLM`` (4.48, the
reference's pin); that part of the reference's behaviour lives in a third-party package that is not available
here, so parity at that boundary is unpinned and checked against an fp32 restatement only.

Parallel layout (one process per GPU, ``world`` ranks): attention heads and the MLP's intermediate features are cut
over the ranks (q/k/v, gate, up by output features; o_proj, down by input features: whole quantisation blocks and
accumulation groups), the residual stream is cut by TOKENS.  Per half-layer a rank normalises and quantises its own
tokens (``rmsnorm_quantize``: the residual add, the norm and the activation quantizer in one kernel), all-gathers
the quantised rows, runs its slice of the block on all tokens, and reduce-scatters the partial outputs back to
token shards -- a reduce-scatter and an all-gather in place of an all-reduce, with the norm and the quantizer done
once per token instead of once per rank.  The batch is cut into ``pieces`` of whole sequences that flow through the
stages one after the other, collectives on a side stream, so that piece i's transfer runs under piece i+1's GEMMs.
With ``world == 1`` the same code runs without any collective.
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import blockquant_ext as ext
from . import kvcache
from .fused import rmsnorm_quantize, softmax_quantize
from .ep_moe import ExpertParallelMoE
from .module import QLinear
from .ops import FP16AccumMatMul, FP32AccumMatMul
from .quantizer import _CudaBlockQuantizer, _QBase


@dataclass
class LlamaArch:
    """Architecture constants (defaults: Llama-3-8B)."""
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    eps: float = 1e-5
    theta: float = 500000.0
    num_experts: int = 0          # > 0: a sparse mixture-of-experts MLP (Mixtral), experts spread over the ranks
    top_k: int = 2


def mixtral_8x7b() -> "LlamaArch":
    """Mixtral-8x7B's constants."""
    return LlamaArch(hidden=4096, layers=32, heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=32000, eps=1e-5,
                     theta=1000000.0, num_experts=8, top_k=2)


def rope_tables(T: int, head_dim: int, theta: float, device, offset: int = 0):
    """cos / sin ``[1, T, head_dim]`` as transformers' ``LlamaRotaryEmbedding`` makes them for an fp16 model:
    computed in fp32 from positions ``offset .. offset + T - 1``, cast to fp16."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    pos = torch.arange(offset, offset + T, dtype=torch.float32, device=device)
    freqs = torch.outer(pos, inv)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.float16)[None], emb.sin().to(torch.float16)[None]


def _same_format(a, b) -> bool:
    if type(a) is not type(b):
        return False
    if isinstance(a, _CudaBlockQuantizer):
        fa, fb = a._format(), b._format()
        return all(getattr(fa, n) == getattr(fb, n) for n, _ in fa._fields_)
    return type(a) is _QBase


def project(lin: QLinear, x: torch.Tensor, input_quantized: bool = False) -> torch.Tensor:
    """``_QBaseLinear.forward`` (src/module.py:42-67) on 2-D fp16 rows with the library's GEMMs: ``ops=None`` (the
    reference's ``F.linear``, fp32 accumulation) runs the tensor-core kernel's fp32 mode.  The non-finite guard of
    the reference is the layer's ``check_finite`` (off in the model: it synchronises the host)."""
    xq = x if input_quantized else lin.aq(x)
    if lin.ops is None:
        y = ext.gemm_fp32_accum(xq, lin.weight, b_is_nk=True, bias=lin.bias)
    else:
        y = lin.ops(xq, lin.weight, lin.bias)
    if lin.check_finite and not torch.isfinite(y).all():
        raise RuntimeError(f"Non-finite output from {type(lin).__name__}({lin.in_features} -> {lin.out_features})")
    return lin.yq(y)


class QLlamaAttention(nn.Module):
    """This rank's heads of the attention block.  Fields as ``PTQ.q_attn`` sets them on the reference's module:
    ``quant_attn_wgt``, ``quant_post_rope_q``, ``quant_k_cache``, ``quant_v_cache``, ``kv_quantizer``,
    ``attn_wgt_quantizer``; projections ``q_proj / k_proj / v_proj / o_proj`` with ``wq / aq / yq / ops``."""

    def __init__(self, arch: LlamaArch, rank: int = 0, world: int = 1, device=None):
        super().__init__()
        if arch.heads % world or arch.kv_heads % world:
            raise ValueError(f"{arch.heads} query / {arch.kv_heads} key-value heads do not divide over {world} ranks")
        self.head_dim = arch.head_dim
        self.num_heads = arch.heads // world                   # local
        self.num_key_value_heads = arch.kv_heads // world      # local
        self.num_key_value_groups = arch.heads // arch.kv_heads
        self.h0, self.kv0 = rank * self.num_heads, rank * self.num_key_value_heads
        kw = dict(bias=False, check_finite=False, device=device, dtype=torch.float16)
        D = arch.head_dim
        self.q_proj = QLinear(arch.hidden, self.num_heads * D, **kw)
        self.k_proj = QLinear(arch.hidden, self.num_key_value_heads * D, **kw)
        self.v_proj = QLinear(arch.hidden, self.num_key_value_heads * D, **kw)
        self.o_proj = QLinear(self.num_heads * D, arch.hidden, **kw)
        self.quant_attn_wgt = self.quant_post_rope_q = self.quant_k_cache = self.quant_v_cache = False
        self.kv_quantizer = None
        self.attn_wgt_quantizer = None
        self.query_chunk = 512                                 # queries per run of a causal prefill (multiple of 128)

    def input_quantizer(self):
        """The one quantizer that serves q/k/v_proj's input when the three agree (every shipped HBQ configuration;
        MX formats with ``qk_mx_round`` round q/k differently from v), else None."""
        a = self.q_proj.aq
        return a if _same_format(a, self.k_proj.aq) and _same_format(a, self.v_proj.aq) else None

    def forward(self, x: torch.Tensor, bsz: int, q_len: int, cos: torch.Tensor, sin: torch.Tensor,
                input_quantized: bool = False) -> torch.Tensor:
        """x ``[bsz * q_len, hidden]`` (already through the shared input quantizer when ``input_quantized``) ->
        this rank's partial o_proj output ``[bsz * q_len, hidden]`` (to be summed over the ranks)."""
        H, Hkv, D, G = self.num_heads, self.num_key_value_heads, self.head_dim, self.num_key_value_groups
        q = project(self.q_proj, x, input_quantized).view(bsz, q_len, H * D)
        k = project(self.k_proj, x, input_quantized).view(bsz, q_len, Hkv * D)
        v = project(self.v_proj, x, input_quantized).view(bsz, q_len, Hkv * D)
        # RoPE, then the post-RoPE Q / K quantizers (src/module.py:158-162), in the cache layout [B, H, T, D]
        if self.quant_post_rope_q and isinstance(self.q_proj.aq, _CudaBlockQuantizer):
            Q = kvcache.write_k_cache(q, H, self.q_proj.aq, cos, sin)
        else:
            Q = kvcache.apply_rope(q.view(bsz, q_len, H, D).transpose(1, 2), cos, sin)
            if self.quant_post_rope_q:
                Q = self.q_proj.aq.q(Q)
        if self.quant_k_cache and isinstance(self.kv_quantizer, _CudaBlockQuantizer):
            K = kvcache.write_k_cache(k, Hkv, self.kv_quantizer, cos, sin)
        else:
            K = kvcache.apply_rope(k.view(bsz, q_len, Hkv, D).transpose(1, 2), cos, sin)
        # V quantised along the token axis (src/module.py:163-168)
        if self.quant_v_cache and isinstance(self.kv_quantizer, _CudaBlockQuantizer):
            V = kvcache.write_v_cache(v, Hkv, self.kv_quantizer)
        else:
            V = v.view(bsz, q_len, Hkv, D).transpose(1, 2)
        # repeat_kv without the copy: the G query heads of a key-value head become rows of one matmul.  A causal
        # prefill is cut into runs of `query_chunk` queries, run c against keys [0, end of run c) only: the keys
        # beyond are masked for every query of the run, their probabilities are zeros and whole quantisation blocks
        # of zeros (runs end on multiples of the 128-key block), so leaving them out changes no value and saves
        # (1 - 1/runs) / 2 of both matmuls and of the softmax sweep.
        aq = self.attn_wgt_quantizer if self.quant_attn_wgt else None
        scale = 1.0 / math.sqrt(D)
        c = self.query_chunk
        if q_len <= c or q_len % c or c % 128:
            Qg = Q.contiguous().view(bsz, Hkv, G * q_len, D)
            scores = torch.matmul(Qg, K.transpose(-1, -2))                  # [B, Hkv, G*T, S] raw q k^T
            P = softmax_quantize(scores, scale, aq, causal=q_len > 1, q_len=q_len, heads=H)
            O = torch.matmul(P, V)                                          # [B, Hkv, G*T, D]
            O = O.view(bsz, H, q_len, D).transpose(1, 2).reshape(bsz * q_len, H * D)
        else:
            Q5 = Q.contiguous().view(bsz, Hkv, G, q_len, D)
            O4 = torch.empty((bsz, q_len, H, D), dtype=Q.dtype, device=Q.device)
            for t0 in range(0, q_len, c):
                t1 = t0 + c
                Qc = Q5[:, :, :, t0:t1].reshape(bsz, Hkv, G * c, D)
                scores = torch.matmul(Qc, K[:, :, :t1].transpose(-1, -2))   # [B, Hkv, G*c, t1]
                P = softmax_quantize(scores, scale, aq, causal=True, q_len=c, heads=H)
                Oc = torch.matmul(P, V[:, :, :t1])                          # [B, Hkv, G*c, D]
                O4[:, t0:t1] = Oc.view(bsz, H, c, D).transpose(1, 2)
            O = O4.view(bsz * q_len, H * D)
        return project(self.o_proj, O)


class QLlamaMLP(nn.Module):
    """This rank's slice of the gated MLP: ``down(silu(gate(x)) * up(x))`` (``QLlamaMLP.forward``,
    src/module.py:547-569; ``quantizer_after_act_fn`` is the optional quantizer of ``quant_before_hadamard``)."""

    def __init__(self, arch: LlamaArch, rank: int = 0, world: int = 1, device=None):
        super().__init__()
        if arch.ffn % (128 * world):
            raise ValueError(f"intermediate size {arch.ffn} does not cut into {world} slices of whole 128-blocks")
        self.f = arch.ffn // world
        self.f0 = rank * self.f
        kw = dict(bias=False, check_finite=False, device=device, dtype=torch.float16)
        self.gate_proj = QLinear(arch.hidden, self.f, **kw)
        self.up_proj = QLinear(arch.hidden, self.f, **kw)
        self.down_proj = QLinear(self.f, arch.hidden, **kw)
        self.quantizer_after_act_fn = None

    def input_quantizer(self):
        a = self.gate_proj.aq
        return a if _same_format(a, self.up_proj.aq) else None

    def forward(self, x: torch.Tensor, input_quantized: bool = False) -> torch.Tensor:
        g = project(self.gate_proj, x, input_quantized)
        u = project(self.up_proj, x, input_quantized)
        if self.quantizer_after_act_fn is None:
            a = kvcache.swiglu_quantize(g, u, self.down_proj.aq)            # silu * up and down_proj.aq in one pass
            return project(self.down_proj, a, input_quantized=True)
        a = self.quantizer_after_act_fn(torch.nn.functional.silu(g)) * u
        return project(self.down_proj, a)


class QLlamaDecoderLayer(nn.Module):
    """Attention + gated MLP, or (``arch.num_experts > 0``, the Mixtral layer) attention + sparse MoE block whose
    experts are ``QMixtralBlockSparseTop2MLP``s (src/module.py:597-622) spread over the ranks."""

    def __init__(self, arch: LlamaArch, rank: int = 0, world: int = 1, device=None, group=None):
        super().__init__()
        self.self_attn = QLlamaAttention(arch, rank, world, device)
        if arch.num_experts > 0:
            self.mlp = None
            self.block_sparse_moe = ExpertParallelMoE(arch.hidden, arch.ffn, arch.num_experts, arch.top_k,
                                                      group=group if world > 1 else None, device=device, dtype=torch.float16,
                                                      local_only=world == 1)
        else:
            self.mlp = QLlamaMLP(arch, rank, world, device)
            self.block_sparse_moe = None
        self.input_layernorm = nn.Parameter(torch.ones(arch.hidden, dtype=torch.float16, device=device))
        self.post_attention_layernorm = nn.Parameter(torch.ones(arch.hidden, dtype=torch.float16, device=device))


class _Piece:
    """One slice of the batch (whole sequences) on its way through the stages."""
    __slots__ = ("bsz", "x", "branch", "act", "full", "part", "ev_compute", "ev_comm")

    def __init__(self, bsz):
        self.bsz = bsz
        self.x = self.branch = self.act = self.full = self.part = None
        self.ev_compute = self.ev_comm = None


class QLlamaModel(nn.Module):
    """Embedding, ``arch.layers`` decoder layers, final norm and a vocabulary-parallel lm_head.

    ``forward(ids)`` returns this rank's logit columns ``[B * T, vocab / world]`` (``gather_logits=True``: all of
    them, for small models).  Weights are drawn N(0, 0.02) per tensor from a seed derived from the tensor's name, in
    full on every rank and then sliced, so every world size holds the same model."""

    def __init__(self, arch: LlamaArch, group=None, device=None, pieces: int = 1, parallel: bool = True):
        """``parallel=False`` builds the whole model on this rank even when a process group exists (the one-GPU
        baseline of a scaling measurement)."""
        super().__init__()
        self.arch = arch
        self.group = group
        on = parallel and dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.pieces = max(1, int(pieces))
        if arch.vocab % self.world:
            raise ValueError(f"vocabulary {arch.vocab} does not divide over {self.world} ranks")
        self.embed_tokens = nn.Embedding(arch.vocab, arch.hidden, device=device, dtype=torch.float16)
        self.layers = nn.ModuleList([QLlamaDecoderLayer(arch, self.rank, self.world, device, group) for _ in range(arch.layers)])
        self.norm = nn.Parameter(torch.ones(arch.hidden, dtype=torch.float16, device=device))
        self.lm_head = nn.Linear(arch.hidden, arch.vocab // self.world, bias=False, device=device, dtype=torch.float16)
        self._comm = None

    # ---- weights ---------------------------------------------------------------------------------
    @staticmethod
    def _draw(name: str, shape, seed: int, device) -> torch.Tensor:
        g = torch.Generator(device=device).manual_seed((zlib.crc32(name.encode()) + seed) & 0x7FFFFFFF)
        return (0.02 * torch.randn(shape, device=device, generator=g)).to(torch.float16)

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        a, dev = self.arch, self.embed_tokens.weight.device
        D = a.head_dim
        self.embed_tokens.weight.copy_(self._draw("embed_tokens", (a.vocab, a.hidden), seed, dev))
        v0 = self.rank * (a.vocab // self.world)
        self.lm_head.weight.copy_(self._draw("lm_head", (a.vocab, a.hidden), seed, dev)[v0:v0 + a.vocab // self.world])
        for i, layer in enumerate(self.layers):
            at, ml = layer.self_attn, layer.mlp
            at.q_proj.weight.copy_(self._draw(f"{i}.q_proj", (a.heads * D, a.hidden), seed, dev)[at.h0 * D:(at.h0 + at.num_heads) * D])
            for nm, lin in (("k_proj", at.k_proj), ("v_proj", at.v_proj)):
                lin.weight.copy_(self._draw(f"{i}.{nm}", (a.kv_heads * D, a.hidden), seed, dev)[at.kv0 * D:(at.kv0 + at.num_key_value_heads) * D])
            at.o_proj.weight.copy_(self._draw(f"{i}.o_proj", (a.hidden, a.heads * D), seed, dev)[:, at.h0 * D:(at.h0 + at.num_heads) * D])
            if ml is None:
                moe = layer.block_sparse_moe
                moe.gate.weight.copy_(self._draw(f"{i}.gate", (a.num_experts, a.hidden), seed, dev))
                for j, ex in enumerate(moe.experts):
                    e = moe.e0 + j
                    ex.w1.weight.copy_(self._draw(f"{i}.experts.{e}.w1", (a.ffn, a.hidden), seed, dev))
                    ex.w3.weight.copy_(self._draw(f"{i}.experts.{e}.w3", (a.ffn, a.hidden), seed, dev))
                    ex.w2.weight.copy_(self._draw(f"{i}.experts.{e}.w2", (a.hidden, a.ffn), seed, dev))
                continue
            for nm, lin in (("gate_proj", ml.gate_proj), ("up_proj", ml.up_proj)):
                lin.weight.copy_(self._draw(f"{i}.{nm}", (a.ffn, a.hidden), seed, dev)[ml.f0:ml.f0 + ml.f])
            ml.down_proj.weight.copy_(self._draw(f"{i}.down_proj", (a.hidden, a.ffn), seed, dev)[:, ml.f0:ml.f0 + ml.f])

    @torch.no_grad()
    def apply_ptq(self, cfg):
        """What ``PTQ.run`` does to the model (src/ptq.py:424-439): inject the quantizers, quantise the weights once,
        set the accumulation operator on every projection of the decoder layers (lm_head stays as it is)."""
        for layer in self.layers:
            cfg.q_attn(layer.self_attn)
            lins = [layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj]
            if layer.mlp is not None:
                cfg.q_mlp(layer.mlp)
                lins += [layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj]
            for lin in lins:
                cfg.static_quant_linear_weight(lin)
                lin.ops = cfg.make_accum_op()
            if layer.block_sparse_moe is not None:
                # q_mixtral_expert (src/ptq.py:292-307) gives w1 and w3 the same input quantizer; block quantisation
                # is per row, so it is applied once per token before the copies travel (the block's `aq`) and the
                # experts' own w1 / w3 input quantizers stay the identity
                moe = layer.block_sparse_moe
                moe.aq = cfg.map_act_quantizer()
                for ex in moe.experts:
                    for lin in (ex.w1, ex.w3, ex.w2):
                        lin.wq = cfg.map_wgt_quantizer()
                        cfg.static_quant_linear_weight(lin)
                        lin.ops = cfg.make_accum_op() or FP32AccumMatMul()
                    ex.w2.aq = cfg.map_act_quantizer()
                    if cfg.quant_before_hadamard:
                        ex.w3.yq = cfg.map_act_quantizer()
                    if cfg.quant_before_silu:
                        ex.w1.yq = cfg.map_act_quantizer()
                    if cfg.quant_before_rms_norm:
                        ex.w2.yq = cfg.map_act_quantizer()
        return self

    # ---- collectives on the side stream -----------------------------------------------------------
    def _comm_stream(self, dev):
        if self._comm is None:
            self._comm = torch.cuda.Stream(dev)
        return self._comm

    def _gather_rows(self, p: _Piece, src: torch.Tensor) -> torch.Tensor:
        """All-gather of token shards ``[n / world, d]`` -> ``[n, d]`` (rank order = token order inside the piece)."""
        if self.world == 1:
            return src
        if not src.is_cuda:
            out = torch.empty((src.shape[0] * self.world, src.shape[1]), dtype=src.dtype)
            dist.all_gather_into_tensor(out, src.contiguous(), group=self.group)
            return out
        cur, side = torch.cuda.current_stream(src.device), self._comm_stream(src.device)
        with torch.cuda.stream(side):
            side.wait_event(p.ev_compute)                     # this piece's producer, not the whole stage
            out = torch.empty((src.shape[0] * self.world, src.shape[1]), dtype=src.dtype, device=src.device)
            dist.all_gather_into_tensor(out, src, group=self.group)
            src.record_stream(side)
            p.ev_comm = torch.cuda.Event()
            p.ev_comm.record(side)
        out.record_stream(cur)
        return out

    def _scatter_rows(self, p: _Piece, src: torch.Tensor) -> torch.Tensor:
        """Reduce-scatter of partial outputs ``[n, d]`` -> this rank's summed token shard ``[n / world, d]``."""
        if self.world == 1:
            return src
        if not src.is_cuda:
            out = torch.empty((src.shape[0] // self.world, src.shape[1]), dtype=src.dtype)
            dist.reduce_scatter_tensor(out, src.contiguous(), group=self.group)
            return out
        cur, side = torch.cuda.current_stream(src.device), self._comm_stream(src.device)
        with torch.cuda.stream(side):
            side.wait_event(p.ev_compute)
            out = torch.empty((src.shape[0] // self.world, src.shape[1]), dtype=src.dtype, device=src.device)
            dist.reduce_scatter_tensor(out, src, group=self.group)
            src.record_stream(side)
            p.ev_comm = torch.cuda.Event()
            p.ev_comm.record(side)
        out.record_stream(cur)
        return out

    @staticmethod
    def _await(p: _Piece):
        """Before a piece's compute stage: its pending collective must have landed."""
        if p.ev_comm is not None:
            torch.cuda.current_stream().wait_event(p.ev_comm)
            p.ev_comm = None

    def _done(self, p: _Piece, t: torch.Tensor):
        """After a piece's compute stage: the point its collective may start from."""
        if self.world > 1 and t.is_cuda:
            p.ev_compute = torch.cuda.Event()
            p.ev_compute.record(torch.cuda.current_stream(t.device))

    # ---- forward -----------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, ids: torch.Tensor, gather_logits: bool = False) -> torch.Tensor:
        a = self.arch
        B, T = ids.shape
        P = self.pieces if B % self.pieces == 0 else 1
        bp = B // P
        n = bp * T
        if n % self.world:
            raise ValueError(f"{n} tokens per piece do not divide over {self.world} ranks")
        shard = n // self.world
        cos, sin = rope_tables(T, a.head_dim, a.theta, ids.device)
        pieces: List[_Piece] = []
        for i in range(P):
            p = _Piece(bp)
            flat = ids[i * bp:(i + 1) * bp].reshape(-1)
            p.x = self.embed_tokens(flat[self.rank * shard:(self.rank + 1) * shard])
            pieces.append(p)

        for layer in self.layers:
            at, ml = layer.self_attn, layer.mlp
            aq_attn, aq_mlp = at.input_quantizer(), (ml.input_quantizer() if ml is not None else None)
            # residual add of the previous branch + input norm + the q/k/v input quantizer, on the token shard
            for p in pieces:
                self._await(p)
                p.act, p.x = rmsnorm_quantize(p.x, layer.input_layernorm, a.eps, aq_attn, residual=p.branch)
                self._done(p, p.act)
            for p in pieces:
                p.full = self._gather_rows(p, p.act)
            for p in pieces:
                self._await(p)
                p.part = at(p.full, p.bsz, T, cos, sin, input_quantized=aq_attn is not None)
                self._done(p, p.part)
            for p in pieces:
                p.branch = self._scatter_rows(p, p.part)
            if layer.block_sparse_moe is not None:
                # sparse MoE on this rank's own tokens: router on the normalised rows, copies to the experts' ranks
                # and back by all-to-all (inside the block); no gather / scatter of rows in this half
                # (two passes over the pieces: the host reads one piece's row counts while the next piece's kernels
                # are already queued, so the read never leaves the GPU without work)
                states = []
                for p in pieces:
                    self._await(p)
                    h, p.x = rmsnorm_quantize(p.x, layer.post_attention_layernorm, a.eps, None, residual=p.branch)
                    states.append(layer.block_sparse_moe.begin(h))
                for p, st in zip(pieces, states):
                    p.branch = layer.block_sparse_moe.finish(st)
                continue
            for p in pieces:
                self._await(p)
                p.act, p.x = rmsnorm_quantize(p.x, layer.post_attention_layernorm, a.eps, aq_mlp, residual=p.branch)
                self._done(p, p.act)
            for p in pieces:
                p.full = self._gather_rows(p, p.act)
            for p in pieces:
                self._await(p)
                p.part = ml(p.full, input_quantized=aq_mlp is not None)
                self._done(p, p.part)
            for p in pieces:
                p.branch = self._scatter_rows(p, p.part)

        outs = []
        for p in pieces:
            self._await(p)
            p.act, p.x = rmsnorm_quantize(p.x, self.norm, a.eps, None, residual=p.branch)
            self._done(p, p.act)
        for p in pieces:
            p.full = self._gather_rows(p, p.act)
        for p in pieces:
            self._await(p)
            logits = torch.nn.functional.linear(p.full, self.lm_head.weight)       # lm_head: untouched by PTQ
            if gather_logits and self.world > 1:
                parts = [torch.empty_like(logits) for _ in range(self.world)]
                dist.all_gather(parts, logits.contiguous(), group=self.group)
                logits = torch.cat(parts, dim=-1)
            outs.append(logits)
        return outs[0] if P == 1 else torch.cat(outs, dim=0)

    def flops_per_token(self) -> float:
        """Multiply-add count x 2 of the linear layers and lm_head for one token (the attention matmuls, which
        grow with the sequence, are counted by ``attention_flops``)."""
        a = self.arch
        D = a.head_dim
        mlp = 3 * a.hidden * a.ffn * (a.top_k if a.num_experts > 0 else 1) + a.hidden * a.num_experts
        per_layer = a.hidden * (a.heads * D + 2 * a.kv_heads * D) + a.heads * D * a.hidden + mlp
        return 2.0 * (a.layers * per_layer + a.hidden * a.vocab)

    def attention_flops(self, B: int, T: int) -> float:
        a = self.arch
        return 4.0 * a.layers * B * a.heads * T * T * a.head_dim
