"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run where the reference checkout is available (its path is the first argument, or the
environment variable ``HBQ_REFERENCE_DIR``)::

    python tests/golden/make_golden.py [/path/to/HBQ]

It imports ``src/quantizer.py`` of the reference unmodified (eager mode:
``use_quant_kernel=False`` / ``activate_dynamo=False``, fp16 CPU tensors) and
stores, as compressed ``.npz`` files of fp16 bit patterns:

* ``exhaustive.npz`` -- the element quantizer ``make_fp_quant`` and the scale
  quantizer ``fp_quant`` over all 65 536 fp16 inputs, and ``floor(log2(x))``
  as evaluated on fp16 tensors;
* ``quantizers.npz`` -- seeded tensors pushed through ``MXFPQuantizer``,
  ``MXINTQuantizer``, ``HBQQuantizer``, ``MXExQuantizer`` and ``VSQQuantizer`` for every format the shipped YAML
  configs use (plus a few corner formats), with the HBQ side outputs
  (``shared_scale``, ``l2_scale``, ``blk_l2_scheme``).

The tests never need the reference at run time: they read these files.
"""
import os
import sys
import warnings

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HBQ_REFERENCE_DIR")
if not REF or not os.path.isdir(os.path.join(REF, "src")):
    raise SystemExit("usage: make_golden.py REFERENCE_DIR (a checkout of SeoLabCornell/HBQ), or set HBQ_REFERENCE_DIR")
sys.path.insert(0, REF)
from src.quantizer import (HBQQuantizer, MXExQuantizer, MXFPQuantizer, MXINTQuantizer,  # noqa: E402
                           VSQQuantizer, fp_quant, make_fp_quant)

HERE = os.path.dirname(os.path.abspath(__file__))
warnings.filterwarnings("ignore")

# name -> (kind, kwargs) ; kwargs are the reference constructor's own names.
FORMATS = {
    # config/hbq_a.yaml, config/hbq_e.yaml (activation / weight), hbq_a_kv.yaml KV4
    "hbq_a_act": ("hbq", dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")),
    "hbq_a_wgt": ("hbq", dict(block_size=128, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="Mix")),
    "hbq_e_act": ("hbq", dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=32, l2_sc_bit=2, l2_scheme="SIG-1")),
    "hbq_e_wgt": ("hbq", dict(block_size=128, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, l2_block_size=32, l2_sc_bit=2, l2_scheme="Mix")),
    "hbq_a_kv4": ("hbq", dict(block_size=128, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=2, l2_scheme="SIG-1")),
    # other L2 schemes / shapes of the same class
    "hbq_pot_b64": ("hbq", dict(block_size=64, ebit=2, mbit=3, sc_ebit=5, sc_mbit=3, l2_block_size=4, l2_sc_bit=1, l2_scheme="PoT")),
    "hbq_int_b32": ("hbq", dict(block_size=32, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, l2_block_size=16, l2_sc_bit=2, l2_scheme="INT")),
    "hbq_fp1": ("hbq", dict(block_size=128, ebit=2, mbit=2, sc_ebit=5, sc_mbit=3, l2_block_size=16, l2_sc_bit=1, l2_scheme="FP1")),
    "hbq_fpm100": ("hbq", dict(block_size=128, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, l2_block_size=8, l2_sc_bit=3, l2_scheme="FP-100")),
    # config/mxfp4.yaml (floor, and round for q/k projections), nvfp4.yaml, mxfp_w4a8.yaml, nvfp_w4a8 (ceil)
    "mxfp4": ("mxfp", dict(block_size=32, ebit=2, mbit=1, sc_ebit=5, sc_mbit=0)),
    "mxfp4_round": ("mxfp", dict(block_size=32, ebit=2, mbit=1, sc_ebit=5, sc_mbit=0, use_round=True)),
    "nvfp4": ("mxfp", dict(block_size=16, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3)),
    "nvfp4_ceil": ("mxfp", dict(block_size=16, ebit=2, mbit=1, sc_ebit=5, sc_mbit=3, use_ceil=True)),
    "nvfp4_e4m3": ("mxfp", dict(block_size=16, ebit=2, mbit=1, sc_ebit=4, sc_mbit=3)),
    "mxfp_a8": ("mxfp", dict(block_size=32, ebit=2, mbit=5, sc_ebit=5, sc_mbit=0)),
    "mxfp6_e2m3": ("mxfp", dict(block_size=32, ebit=2, mbit=3, sc_ebit=5, sc_mbit=0)),
    "mxfp8_e4m3": ("mxfp", dict(block_size=32, ebit=4, mbit=3, sc_ebit=8, sc_mbit=0)),
    # config/mxint8.yaml, mxint_w4a8.yaml
    "mxint8": ("mxint", dict(nbit=8, sc_ebit=8, sc_mbit=0, block_size=32)),
    "mxint4": ("mxint", dict(nbit=4, sc_ebit=8, sc_mbit=0, block_size=32)),
    "mxint8_fpscale": ("mxint", dict(nbit=8, sc_ebit=5, sc_mbit=3, block_size=16)),
    # the two remaining quantizer classes of src/quantizer.py (no shipped YAML selects them)
    "mxex_m3": ("mxex", dict(block_size=16, l2_block_size=2, sc_bit=8, l2_sc_bit=1, mbit=3)),
    "mxex_m5_l4": ("mxex", dict(block_size=32, l2_block_size=4, sc_bit=8, l2_sc_bit=1, mbit=5)),
    "vsq4": ("vsq", dict(nbit=4, block_size=16, sc_mbit=4)),
    "vsq8_b32": ("vsq", dict(nbit=8, block_size=32, sc_mbit=6)),
}


def make_quantizer(kind, kw):
    if kind == "hbq":
        return HBQQuantizer(keep_l2_scale=True, use_quant_kernel=False, **kw)
    if kind == "mxfp":
        return MXFPQuantizer(activate_dynamo=False, **kw)
    if kind == "mxex":
        return MXExQuantizer(**kw)
    if kind == "vsq":
        return VSQQuantizer(**kw)
    return MXINTQuantizer(**kw)


def inputs():
    """Seeded fp16 test tensors; shapes include a ragged K and all-zero blocks."""
    g = torch.Generator().manual_seed(1234)
    out = {}
    x = torch.randn(24, 512, generator=g)
    x[:, torch.randperm(512, generator=g)[:5]] *= 20
    out["act"] = x
    out["wgt"] = 0.02 * torch.randn(24, 512, generator=g)
    torch.manual_seed(99)
    out["studt"] = 0.5 * torch.distributions.StudentT(3.0).sample((16, 600))   # ragged K
    out["tiny"] = 2e-5 * torch.randn(8, 256, generator=g)
    out["huge"] = 4000 * torch.randn(8, 256, generator=g)
    short = torch.randn(4, 40, generator=g)                                   # K < block for most
    out["short"] = short
    res = {}
    for k, v in out.items():
        v = v.to(torch.float16)
        v[0, : min(v.shape[1], 160)] = 0
        res[k] = v
    return res


def bits(t):
    return t.contiguous().numpy().view(np.uint16)


def main():
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    allh = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16)
    finite = torch.isfinite(allh)
    ex = {"finite": finite.numpy()}
    xs = allh[finite]
    for e, m in [(2, 1), (2, 2), (2, 3), (2, 5), (3, 2), (4, 3), (5, 2)]:
        ex[f"elem_e{e}m{m}"] = bits(make_fp_quant(e, m)(xs))
    for se, sm in [(5, 3), (4, 3)]:
        for ceil in (0, 1):
            for sub in (0, 1):
                ex[f"scale_e{se}m{sm}_ceil{ceil}_sub{sub}"] = bits(
                    fp_quant(xs, se, sm, allow_subnormal=bool(sub), use_ceil=bool(ceil)))
    pos = allh[(allh > 0) & finite]
    ex["floor_log2_pos"] = torch.floor(torch.log2(pos)).to(torch.int8).numpy()
    np.savez_compressed(os.path.join(HERE, "exhaustive.npz"), **ex)

    q = {}
    ins = inputs()
    for k, v in ins.items():
        q[f"in/{k}"] = bits(v)
    for name, (kind, kw) in FORMATS.items():
        quant = make_quantizer(kind, kw)
        for k, v in ins.items():
            y = quant.q(v.clone())
            assert y.dtype == torch.float16 and y.shape == v.shape
            q[f"out/{name}/{k}/deq"] = bits(y)
            if kind == "hbq":
                q[f"out/{name}/{k}/scale"] = bits(quant.shared_scale)
                q[f"out/{name}/{k}/l2"] = quant.l2_scale.numpy().astype(np.uint8)
                q[f"out/{name}/{k}/scheme"] = quant.blk_l2_scheme.numpy().astype(np.uint8)
    np.savez_compressed(os.path.join(HERE, "quantizers.npz"), **q)
    import json
    with open(os.path.join(HERE, "formats.json"), "w") as fh:
        json.dump({k: {"kind": v[0], **v[1]} for k, v in FORMATS.items()}, fh, indent=1)
    for f in ("exhaustive.npz", "quantizers.npz", "formats.json"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
