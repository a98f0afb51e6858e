"""YAML quantization config -> quantizer / GEMM-operator objects, with the keys and defaults of
the reference's ``PTQ`` (src/ptq.py:29-105) and its factory methods (src/ptq.py:107-257,
384-404).  The reference's model plumbing (Hugging Face module patching) is not reproduced;
``apply_to_linear`` performs its per-layer steps on one ``QLinear``.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .module import QLinear
from .ops import FP16AccumMatMul
from .quantizer import HBQQuantizer, MXExQuantizer, MXFPQuantizer, MXINTQuantizer, VSQQuantizer, _QBase


def load_quant_config(path: str) -> Dict[str, Any]:
    import yaml
    with open(path, "r") as fh:
        return yaml.full_load(fh)


class PTQConfig:
    """Parsed quantization YAML (the second YAML of a reference run, config/README.md)."""

    def __init__(self, quant_config: Dict[str, Any]):
        # not a YAML field: keep every statically quantised weight also as packed codes in the decode GEMM's tile
        # order (QLinear.prepare_decode), so that decode-sized batches stream 0.56 B per weight
        self.pack_for_decode = False
        self.quant_config = quant_config
        q = quant_config.get("quantization", {})
        b = quant_config.get("block_quant", {})
        acc = quant_config.get("accumulation", {})
        self.xqtype = q["xqtype"]
        self.wqtype = q["wqtype"]
        self.a_ebit = b.get("act_ebit", 0)
        self.a_mbit = b.get("act_mbit", 0)
        self.a_sc_ebit = b.get("act_sc_ebit", 0)
        self.a_sc_mbit = b.get("act_sc_mbit", 8)
        self.a_block_size = b.get("act_block_size", 32)
        self.kv_block_size = b.get("kv_block_size", self.a_block_size)
        self.a_per_tensor_scale = b.get("act_per_tensor_scale", False)
        self.w_ebit = b.get("wgt_ebit", 0)
        self.w_mbit = b.get("wgt_mbit", 0)
        self.w_sc_ebit = b.get("wgt_sc_ebit", 0)
        self.w_sc_mbit = b.get("wgt_sc_mbit", 8)
        self.w_block_size = b.get("wgt_block_size", 32)
        self.w_per_tensor_scale = b.get("wgt_per_tensor_scale", False)
        self.scale_allow_subnormal = b.get("scale_allow_subnormal", True)
        # MicroExponent quantization (src/ptq.py:60-61)
        self.a_sc_bit = b.get("act_sc_bit", 8)
        self.w_sc_bit = b.get("wgt_sc_bit", 8)
        self.qk_mx_round = b.get("qk_mx_round", False)
        self.act_scale_use_ceil = b.get("act_scale_use_ceil", False)
        self.wgt_scale_use_ceil = b.get("wgt_scale_use_ceil", False)
        self.wgt_l2_sc_bit = b.get("wgt_l2_sc_bit", 1)
        self.wgt_l2_block_size = b.get("wgt_l2_block_size", 4)
        self.wgt_l2_scheme = b.get("wgt_l2_scheme", "PoT")
        self.act_l2_sc_bit = b.get("act_l2_sc_bit", 1)
        self.act_l2_block_size = b.get("act_l2_block_size", 4)
        self.act_l2_scheme = b.get("act_l2_scheme", "PoT")
        self.quant_before_hadamard = q.get("quant_before_hadamard", False)
        self.quant_before_silu = q.get("quant_before_silu", False)
        self.quant_before_rms_norm = q.get("quant_before_rms_norm", False)
        self.quant_embedding_layer = q.get("quant_embedding_layer", False)
        self.quant_output_layer = q.get("quant_output_layer", False)
        self.quant_attn_wgt = q.get("quant_attn_wgt", False)
        self.quant_post_rope_q = q.get("quant_post_rope_q", False)
        self.quant_4b_kv = q.get("quant_4b_kv", False)
        self.quant_k_cache = q.get("quant_k_cache", False)
        self.quant_v_cache = q.get("quant_v_cache", False)
        self.quant_post_rope_qk = q.get("quant_post_rope_qk", False)        # read and unused, as in the reference
        self.quant_attn_wgt_use_quant_kernel = q.get("quant_attn_wgt_use_quant_kernel", True)
        self.accumulation_type = acc.get("type", "fp32")
        self.accumulation_group_size = acc.get("group_size", 128)
        self.accumulation_quant_block_size = acc.get("quant_block_size", 16)

    # ---- src/ptq.py:107-157 ----
    def map_wgt_quantizer(self, use_round: bool = False):
        if self.wqtype == "mxfp":
            return MXFPQuantizer(ebit=self.w_ebit, mbit=self.w_mbit, sc_ebit=self.w_sc_ebit, sc_mbit=self.w_sc_mbit,
                                 block_size=self.w_block_size, per_tensor_scale=self.w_per_tensor_scale,
                                 scale_allow_subnormal=self.scale_allow_subnormal, use_round=use_round,
                                 use_ceil=self.wgt_scale_use_ceil)
        if self.wqtype == "mxint":
            return MXINTQuantizer(nbit=self.w_mbit, sc_ebit=self.w_sc_ebit, sc_mbit=self.w_sc_mbit,
                                  block_size=self.w_block_size, scale_allow_subnormal=self.scale_allow_subnormal)
        if self.wqtype == "mxex":
            return MXExQuantizer(sc_bit=self.w_sc_bit, l2_sc_bit=self.wgt_l2_sc_bit, mbit=self.w_mbit,
                                 block_size=self.w_block_size, l2_block_size=self.wgt_l2_block_size)
        if self.wqtype == "vsq":
            return VSQQuantizer(nbit=self.w_mbit, block_size=self.w_block_size, sc_mbit=self.w_sc_mbit)
        if self.wqtype == "hbq":
            return HBQQuantizer(ebit=self.w_ebit, mbit=self.w_mbit, sc_ebit=self.w_sc_ebit, sc_mbit=self.w_sc_mbit,
                                block_size=self.w_block_size, scale_allow_subnormal=self.scale_allow_subnormal,
                                l2_block_size=self.wgt_l2_block_size, l2_sc_bit=self.wgt_l2_sc_bit,
                                l2_scheme=self.wgt_l2_scheme)
        if self.wqtype == "none":
            return _QBase()
        raise AssertionError(f"Invalid weight quantizer type: {self.wqtype}")

    # ---- src/ptq.py:159-212 ----
    def map_act_quantizer(self, use_round: bool = False, use_quant_kernel: bool = True):
        """``use_quant_kernel`` is accepted as in the reference and has no effect: there is one
        implementation, the CUDA kernel."""
        if self.xqtype == "mxfp":
            return MXFPQuantizer(ebit=self.a_ebit, mbit=self.a_mbit, sc_ebit=self.a_sc_ebit, sc_mbit=self.a_sc_mbit,
                                 block_size=self.a_block_size, per_tensor_scale=self.a_per_tensor_scale,
                                 scale_allow_subnormal=self.scale_allow_subnormal, use_round=use_round,
                                 use_ceil=self.act_scale_use_ceil)
        if self.xqtype == "mxint":
            return MXINTQuantizer(nbit=self.a_mbit, sc_ebit=self.a_sc_ebit, sc_mbit=self.a_sc_mbit,
                                  block_size=self.a_block_size, scale_allow_subnormal=self.scale_allow_subnormal)
        if self.xqtype == "mxex":
            return MXExQuantizer(sc_bit=self.a_sc_bit, l2_sc_bit=self.act_l2_sc_bit, mbit=self.a_mbit,
                                 block_size=self.a_block_size, l2_block_size=self.act_l2_block_size)
        if self.xqtype == "vsq":
            return VSQQuantizer(nbit=self.a_mbit, block_size=self.a_block_size, sc_mbit=self.a_sc_mbit)
        if self.xqtype == "hbq":
            return HBQQuantizer(ebit=self.a_ebit, mbit=self.a_mbit, sc_ebit=self.a_sc_ebit, sc_mbit=self.a_sc_mbit,
                                block_size=self.a_block_size, scale_allow_subnormal=self.scale_allow_subnormal,
                                l2_block_size=self.act_l2_block_size, l2_sc_bit=self.act_l2_sc_bit,
                                l2_scheme=self.act_l2_scheme)
        if self.xqtype == "none":
            return _QBase()
        raise AssertionError(f"Invalid activation quantizer type: {self.xqtype}")

    # ---- src/ptq.py:214-257: 4-bit KV quantizer with the activation's scale settings ----
    def map_4b_kv_quantizer(self, use_round: bool = False):
        if self.xqtype == "mxfp":
            return MXFPQuantizer(ebit=2, mbit=1, sc_ebit=self.a_sc_ebit, sc_mbit=self.a_sc_mbit,
                                 block_size=self.kv_block_size, per_tensor_scale=self.a_per_tensor_scale,
                                 scale_allow_subnormal=self.scale_allow_subnormal, use_round=use_round,
                                 use_ceil=self.act_scale_use_ceil)
        if self.xqtype == "mxint":
            return MXINTQuantizer(nbit=4, sc_ebit=self.a_sc_ebit, sc_mbit=self.a_sc_mbit,
                                  block_size=self.kv_block_size, scale_allow_subnormal=self.scale_allow_subnormal)
        if self.xqtype == "hbq":
            return HBQQuantizer(ebit=2, mbit=1, sc_ebit=self.a_sc_ebit, sc_mbit=self.a_sc_mbit,
                                block_size=self.kv_block_size, scale_allow_subnormal=self.scale_allow_subnormal,
                                l2_block_size=self.act_l2_block_size, l2_sc_bit=self.act_l2_sc_bit,
                                l2_scheme=self.act_l2_scheme)
        if self.xqtype == "none":
            return _QBase()
        raise AssertionError(f"Invalid activation quantizer type: {self.xqtype}")

    def map_kv_quantizer(self):
        """KV-cache quantizer as src/ptq.py:267-270 chooses it."""
        if self.quant_4b_kv:
            return self.map_4b_kv_quantizer(use_round=self.qk_mx_round)
        return self.map_act_quantizer(use_round=self.qk_mx_round)

    # ---- src/ptq.py:259-290: quantizers of one attention block ----
    def q_attn(self, module):
        """``module`` has ``q_proj / k_proj / v_proj / o_proj`` (``QLinear``-like: fields ``wq``, ``aq``,
        ``yq``) and receives the switches and quantizers the reference's attention forwards read:
        ``quant_attn_wgt``, ``quant_post_rope_q``, ``quant_k_cache``, ``quant_v_cache``,
        ``kv_quantizer``, ``attn_wgt_quantizer``."""
        module.quant_attn_wgt = self.quant_attn_wgt
        module.quant_post_rope_q = self.quant_post_rope_q
        module.quant_k_cache = self.quant_k_cache
        module.quant_v_cache = self.quant_v_cache
        module.kv_quantizer = self.map_kv_quantizer()
        module.attn_wgt_quantizer = (self.map_act_quantizer(use_round=self.qk_mx_round,
                                                            use_quant_kernel=self.quant_attn_wgt_use_quant_kernel)
                                     if self.quant_attn_wgt else None)
        for proj in (module.q_proj, module.k_proj):
            proj.wq = self.map_wgt_quantizer(use_round=self.qk_mx_round)
            proj.aq = self.map_act_quantizer(use_round=self.qk_mx_round)
        module.v_proj.wq = self.map_wgt_quantizer()
        module.v_proj.aq = self.map_act_quantizer()
        module.o_proj.wq = self.map_wgt_quantizer()
        module.o_proj.aq = self.map_act_quantizer()
        if self.quant_before_rms_norm:
            module.o_proj.yq = self.map_act_quantizer()

    # ---- src/ptq.py:292-324: quantizers of one gated MLP (names of the Llama / Qwen2 block, or of a Mixtral expert) ----
    def _q_gated(self, module, gate: str, up: str, down: str):
        u, g, d = getattr(module, up), getattr(module, gate), getattr(module, down)
        u.wq, u.aq = self.map_wgt_quantizer(), self.map_act_quantizer()
        if self.quant_before_hadamard:
            u.yq = self.map_act_quantizer()
            module.quantizer_after_act_fn = self.map_act_quantizer(None)
        g.wq, g.aq = self.map_wgt_quantizer(), self.map_act_quantizer()
        if self.quant_before_silu:
            g.yq = self.map_act_quantizer()
        d.wq, d.aq = self.map_wgt_quantizer(), self.map_act_quantizer()
        if self.quant_before_rms_norm:
            d.yq = self.map_act_quantizer()

    def q_mlp(self, module):
        self._q_gated(module, "gate_proj", "up_proj", "down_proj")

    def q_mixtral_expert(self, module):
        self._q_gated(module, "w1", "w3", "w2")

    @torch.no_grad()
    def static_quant_linear_weight(self, linear):
        """``weight.data = linear.wq(weight)`` (src/ptq.py:337-358; the reference's row chunking only bounds
        the memory of its eager quantizer, which expands tensors 4-8x, and is not needed here)."""
        if self.pack_for_decode and self.accumulation_type == "fp32" and hasattr(linear, "prepare_decode") and \
                linear.weight.is_cuda and hasattr(linear.wq, "quantize_packed"):
            # one pass gives the packed codes and the fp16 tensor; the packed form also serves decode-sized batches
            try:
                linear.pack_weight(linear.wq)
                linear.prepare_decode()
                return
            except NotImplementedError:
                pass
        linear.weight.data = linear.wq(linear.weight.data)

    # ---- src/ptq.py:384-404 ----
    def make_accum_op(self) -> Optional[FP16AccumMatMul]:
        if self.accumulation_type == "fp32":
            return None
        if self.accumulation_type == "fp16":
            return FP16AccumMatMul(group_size=self.accumulation_group_size)
        if self.accumulation_type == "fp16_quant":
            return FP16AccumMatMul(group_size=self.accumulation_group_size,
                                   quant_block_size=self.accumulation_quant_block_size)
        raise ValueError(f"Invalid accumulation type: {self.accumulation_type}")

    # which YAML switch gives a projection an output quantizer ``yq`` (src/ptq.py:287-324)
    _YQ_SWITCH = {"o_proj": "quant_before_rms_norm", "down_proj": "quant_before_rms_norm", "w2": "quant_before_rms_norm",
                  "up_proj": "quant_before_hadamard", "w3": "quant_before_hadamard",
                  "gate_proj": "quant_before_silu", "w1": "quant_before_silu"}

    @torch.no_grad()
    def apply_to_linear(self, linear: QLinear, qk_proj: bool = False, role: Optional[str] = None) -> QLinear:
        """Inject quantizers, fake-quantise the weight once and set the GEMM operator: what
        inject_quantizers / static_quant_wgt / replace_accum_kernel do to one layer
        (src/ptq.py:259-324, 337-404).  ``qk_proj`` selects the q/k-projection rounding rule;
        ``role`` (the projection's name in the reference's blocks: ``o_proj``, ``up_proj``,
        ``gate_proj``, ``down_proj``, ``w1``/``w2``/``w3``) adds the output quantizer ``yq`` when the
        matching ``quant_before_*`` switch is on."""
        use_round = self.qk_mx_round if qk_proj else False
        linear.wq = self.map_wgt_quantizer(use_round=use_round)
        linear.aq = self.map_act_quantizer(use_round=use_round)
        switch = self._YQ_SWITCH.get(role) if role is not None else None
        if role is not None and switch is None and role not in ("q_proj", "k_proj", "v_proj"):
            raise ValueError(f"unknown projection role: {role}")
        if switch is not None and getattr(self, switch):
            linear.yq = self.map_act_quantizer()
        linear.weight.data = linear.wq(linear.weight.data)
        linear.ops = self.make_accum_op()
        return linear
