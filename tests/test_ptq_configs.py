"""CPU: the YAML contract.  Every quantisation YAML the reference ships maps to the same quantizer
objects through ``hbq_b200.PTQConfig`` as through the reference's own ``PTQ`` (fixture made by
tests/golden/make_ptq_golden.py), and the reference's ``src/ptq.py``, imported with the two import
lines swapped as a maintainer would, builds ``hbq_b200`` objects with the same fields."""
import importlib
import json
import logging
import os
import sys
import types

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

with open(os.path.join(HERE, "golden", "ptq_configs.json")) as _fh:
    GOLDEN = json.load(_fh)


def fields(q):
    return {k: v for k, v in vars(q).items()
            if not k.startswith("_") and k != "training" and isinstance(v, (int, float, bool, str))}


def same(q, want):
    """Class name and every constructor field the reference object carries."""
    assert type(q).__name__ == want["class"], (type(q).__name__, want["class"])
    got = fields(q)
    for k, v in want["fields"].items():
        assert k in got and got[k] == v, (type(q).__name__, k, got.get(k), v)


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_every_shipped_quantisation_yaml(name):
    import hbq_b200 as H
    rec = GOLDEN[name]
    cfg = H.PTQConfig(rec["config"])
    same(cfg.map_wgt_quantizer(), rec["wgt"])
    same(cfg.map_wgt_quantizer(use_round=True), rec["wgt_round"])
    same(cfg.map_act_quantizer(), rec["act"])
    same(cfg.map_act_quantizer(use_round=True), rec["act_round"])
    if "kv4" in rec:
        same(cfg.map_4b_kv_quantizer(use_round=cfg.qk_mx_round), rec["kv4"])
    assert [cfg.accumulation_type, cfg.accumulation_group_size, cfg.accumulation_quant_block_size] == rec["accumulation"]
    for k, v in rec["switches"].items():
        assert getattr(cfg, k) == v, (k, getattr(cfg, k), v)
    op = cfg.make_accum_op()
    if rec["accumulation"][0] == "fp32":
        assert op is None
    else:
        assert isinstance(op, H.FP16AccumMatMul) and op.group_size == rec["accumulation"][1]
        assert op.quant_block_size == (rec["accumulation"][2] if rec["accumulation"][0] == "fp16_quant" else None)


def test_vsq_and_mxex_types():
    import hbq_b200 as H
    c = H.PTQConfig({"quantization": {"xqtype": "mxex", "wqtype": "vsq"},
                     "block_quant": {"act_mbit": 5, "act_sc_bit": 6, "act_l2_sc_bit": 1, "act_l2_block_size": 2,
                                     "act_block_size": 16, "wgt_mbit": 4, "wgt_block_size": 16, "wgt_sc_mbit": 4}})
    a, w = c.map_act_quantizer(), c.map_wgt_quantizer()
    assert isinstance(a, H.MXExQuantizer) and (a.sc_bit, a.mbit, a.l2_block_size, a.block_size) == (6, 5, 2, 16)
    assert isinstance(w, H.VSQQuantizer) and (w.nbit, w.block_size, w.sc_mbit) == (4, 16, 4)
    with pytest.raises(AssertionError):
        H.PTQConfig({"quantization": {"xqtype": "int3", "wqtype": "none"}}).map_act_quantizer()


def _reference_dir():
    """A checkout of the reference: HBQ_REFERENCE_DIR, else a directory `reference` beside this repository."""
    for cand in (os.environ.get("HBQ_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "src", "ptq.py")):
            return cand
    return None


def test_reference_ptq_runs_with_the_import_swap():
    """`from src.quantizer import ...` and `from src.ops import FP16AccumMatMul` of the reference's
    src/ptq.py and src/module.py resolve to hbq_b200; its PTQ then builds hbq_b200 objects, injects them
    into attention / MLP stand-ins through its own q_attn / q_mlp, and its replace_accum_kernel installs
    hbq_b200's operator."""
    ref = _reference_dir()
    if ref is None:
        pytest.skip("no checkout of the reference (set HBQ_REFERENCE_DIR)")
    pytest.importorskip("transformers")
    import torch.nn as nn
    import hbq_b200 as H

    saved = {k: sys.modules.get(k) for k in ("src", "src.quantizer", "src.ops", "src.module", "src.ptq", "src.compat",
                                             "blockquant_ext")}
    qmod = types.ModuleType("src.quantizer")
    for n in ("_QBase", "MXFPQuantizer", "MXINTQuantizer", "HBQQuantizer", "MXExQuantizer", "VSQQuantizer"):
        setattr(qmod, n, getattr(H, n))
    omod = types.ModuleType("src.ops")
    omod.FP16AccumMatMul = H.FP16AccumMatMul
    sys.path.insert(0, ref)
    try:
        for k in saved:
            sys.modules.pop(k, None)
        sys.modules["src.quantizer"] = qmod
        sys.modules["src.ops"] = omod
        sys.modules["blockquant_ext"] = H.blockquant_ext
        try:
            ptq = importlib.import_module("src.ptq")
        except ImportError as e:                      # the installed transformers lacks a class the reference's module.py needs
            pytest.skip(f"reference src/ptq.py does not import here: {e}")
        for name, rec in sorted(GOLDEN.items()):
            class Model(nn.Module):
                config = None
            p = ptq.PTQ(rec["config"], Model(), None, logging.getLogger("ptq"))
            ours = H.PTQConfig(rec["config"])
            for got, want in ((p.map_wgt_quantizer(), ours.map_wgt_quantizer()),
                              (p.map_act_quantizer(use_round=True), ours.map_act_quantizer(use_round=True))):
                assert type(got) is type(want) and type(got).__module__.startswith("hbq_b200"), (name, type(got))
                assert fields(got) == fields(want), (name, fields(got), fields(want))
            if name == "hbq_a_kv.yaml":
                # the reference's own injection over stand-ins for its attention / MLP modules
                lin = ptq._QBaseLinear
                attn = types.SimpleNamespace(q_proj=lin(8, 8), k_proj=lin(8, 8), v_proj=lin(8, 8), o_proj=lin(8, 8))
                mlp = types.SimpleNamespace(gate_proj=lin(8, 8), up_proj=lin(8, 8), down_proj=lin(8, 8))
                p.q_attn(attn)
                p.q_mlp(mlp)
                mine_a = types.SimpleNamespace(q_proj=H.QLinear(8, 8), k_proj=H.QLinear(8, 8), v_proj=H.QLinear(8, 8),
                                               o_proj=H.QLinear(8, 8))
                mine_m = types.SimpleNamespace(gate_proj=H.QLinear(8, 8), up_proj=H.QLinear(8, 8), down_proj=H.QLinear(8, 8))
                ours.q_attn(mine_a)
                ours.q_mlp(mine_m)
                assert isinstance(attn.kv_quantizer, H.HBQQuantizer) and attn.kv_quantizer.mbit == 1
                assert fields(attn.kv_quantizer) == fields(mine_a.kv_quantizer)
                assert fields(attn.attn_wgt_quantizer) == fields(mine_a.attn_wgt_quantizer)
                for a, b in ((attn, mine_a), (mlp, mine_m)):
                    for pn, proj in vars(a).items():
                        if isinstance(proj, nn.Linear):
                            for role in ("wq", "aq", "yq"):
                                ga, gb = getattr(proj, role), getattr(getattr(b, pn), role)
                                assert type(ga) is type(gb) and fields(ga) == fields(gb), (pn, role)
                for k in ("quant_attn_wgt", "quant_post_rope_q", "quant_k_cache", "quant_v_cache"):
                    assert getattr(attn, k) == getattr(mine_a, k) is True
            if rec["accumulation"][0] != "fp32":
                layer = type("LlamaDecoderLayer", (nn.Module,), {})
                # replace_accum_kernel walks decoder layers by class: give it one of the class it imported
                dec = ptq.LlamaDecoderLayer.__new__(ptq.LlamaDecoderLayer)
                nn.Module.__init__(dec)
                dec.proj = ptq._QBaseLinear(8, 8)
                model = nn.Module()
                model.layer = dec
                p.model = model
                p.replace_accum_kernel()
                assert isinstance(dec.proj.ops, H.FP16AccumMatMul)
                assert dec.proj.ops.group_size == rec["accumulation"][1]
                del layer
    finally:
        sys.path.remove(ref)
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v
