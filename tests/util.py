"""Helpers shared by the tests: golden-file access and format translation."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")


def load_formats():
    with open(os.path.join(GOLDEN, "formats.json")) as fh:
        return json.load(fh)


def load_npz(name):
    return np.load(os.path.join(GOLDEN, name))


def oracle_format(O, spec):
    """formats.json entry (reference constructor kwargs) -> oracle Format."""
    kind = spec["kind"]
    if kind == "hbq":
        return O.Format(O.KIND_HBQ, spec["ebit"], spec["mbit"], spec["sc_ebit"], spec["sc_mbit"], spec["block_size"],
                        l2_block_size=spec["l2_block_size"], l2_sc_bit=spec["l2_sc_bit"], l2_scheme=spec["l2_scheme"])
    if kind == "mxfp":
        return O.Format(O.KIND_MXFP, spec["ebit"], spec["mbit"], spec["sc_ebit"], spec["sc_mbit"], spec["block_size"],
                        use_round=spec.get("use_round", False), use_ceil=spec.get("use_ceil", False),
                        per_tensor_scale=spec.get("per_tensor_scale", False))
    if kind == "mxex":
        return O.Format(O.KIND_MXEX, 0, spec["mbit"], spec["sc_bit"], 0, spec["block_size"],
                        l2_block_size=spec["l2_block_size"], l2_sc_bit=spec["l2_sc_bit"])
    if kind == "vsq":
        return O.Format(O.KIND_VSQ, 0, spec["nbit"], 0, spec["sc_mbit"], spec["block_size"])
    return O.Format(O.KIND_MXINT, 0, spec["nbit"], spec["sc_ebit"], spec["sc_mbit"], spec["block_size"])


def make_quantizer(spec, **extra):
    """formats.json entry -> hbq_b200 quantizer (same kwargs as the reference constructors)."""
    import hbq_b200 as H
    kw = {k: v for k, v in spec.items() if k != "kind"}
    kw.update(extra)
    if spec["kind"] == "mxex":
        return H.MXExQuantizer(**kw)
    if spec["kind"] == "vsq":
        return H.VSQQuantizer(**kw)
    if spec["kind"] == "hbq":
        return H.HBQQuantizer(**kw)
    if spec["kind"] == "mxfp":
        return H.MXFPQuantizer(**kw)
    return H.MXINTQuantizer(**kw)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def seeded_inputs(kind, rows, K, seed=0):
    """Synthetic tensors with the value distributions of the benchmark configurations:
    'act' N(0,1) with 1% outlier channels x20; 'wgt' N(0, 0.02); 'studt' 0.5*Student-t(3)."""
    rng = np.random.default_rng(seed)
    if kind == "act":
        x = rng.standard_normal((rows, K)).astype(np.float32)
        cols = rng.permutation(K)[: max(1, K // 100)]
        x[:, cols] *= 20
    elif kind == "wgt":
        x = 0.02 * rng.standard_normal((rows, K)).astype(np.float32)
    elif kind == "studt":
        x = 0.5 * rng.standard_t(3, size=(rows, K)).astype(np.float32)
    else:
        raise ValueError(kind)
    return x.astype(np.float16)
