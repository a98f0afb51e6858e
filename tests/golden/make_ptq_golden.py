"""Writes ptq_configs.json: for every quantisation YAML the reference ships (config/*.yaml with a
``quantization`` section) the parsed YAML and the quantizer objects the reference's own ``PTQ``
(src/ptq.py:29-257, 384-404) builds from it -- class name and constructor fields of the weight,
activation and 4-bit KV quantizers (with and without the q/k rounding rule) and the accumulation
settings.  tests/test_ptq_configs.py holds ``hbq_b200.PTQConfig`` to these.

    python tests/golden/make_ptq_golden.py [REFERENCE_DIR]

REFERENCE_DIR (or the environment variable HBQ_REFERENCE_DIR) is a checkout of SeoLabCornell/HBQ;
the reference code is imported unmodified and runs on CPU.
"""
import glob
import json
import logging
import os
import sys

import yaml

HERE = os.path.dirname(os.path.abspath(__file__))


def fields(q):
    d = {k: v for k, v in vars(q).items()
         if not k.startswith("_") and k != "training" and isinstance(v, (int, float, bool, str))}
    return {"class": type(q).__name__, "fields": d}


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HBQ_REFERENCE_DIR")
    if not ref or not os.path.isdir(ref):
        raise SystemExit("usage: make_ptq_golden.py REFERENCE_DIR (or set HBQ_REFERENCE_DIR)")
    sys.path.insert(0, ref)
    import src.ptq as P

    class Model:
        config = None

    out = {}
    for path in sorted(glob.glob(os.path.join(ref, "config", "*.yaml"))):
        with open(path) as fh:
            cfg = yaml.full_load(fh)
        if not isinstance(cfg, dict) or "quantization" not in cfg:
            continue
        p = P.PTQ(cfg, Model(), None, logging.getLogger("ptq"))
        rec = {"config": cfg,
               "wgt": fields(p.map_wgt_quantizer()), "wgt_round": fields(p.map_wgt_quantizer(use_round=True)),
               "act": fields(p.map_act_quantizer()), "act_round": fields(p.map_act_quantizer(use_round=True)),
               "accumulation": [p.accumulation_type, p.accumulation_group_size, p.accumulation_quant_block_size],
               "switches": {k: getattr(p, k) for k in (
                   "quant_before_hadamard", "quant_before_silu", "quant_before_rms_norm", "quant_embedding_layer",
                   "quant_output_layer", "quant_attn_wgt", "quant_post_rope_q", "quant_4b_kv", "quant_k_cache",
                   "quant_v_cache", "quant_attn_wgt_use_quant_kernel", "qk_mx_round", "kv_block_size",
                   "scale_allow_subnormal", "a_sc_bit", "w_sc_bit")}}
        if p.xqtype in ("mxfp", "mxint", "hbq", "none"):
            rec["kv4"] = fields(p.map_4b_kv_quantizer(use_round=p.qk_mx_round))
        out[os.path.basename(path)] = rec
    with open(os.path.join(HERE, "ptq_configs.json"), "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)
    print(f"{len(out)} quantisation YAMLs -> ptq_configs.json")


if __name__ == "__main__":
    main()
