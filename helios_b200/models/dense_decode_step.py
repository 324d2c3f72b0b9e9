"""A whole decode step of the dense GQA decoder in one persistent kernel
(``csrc/decode_step.cu``), for steps of at most eight requests with one token each.

The model's forward pass (``DecoderModel.forward``; python/helios/exec/model.py:465-496 in
the reference) asks the plan's ``fused_steps`` first: each may take the step over whole or
decline.  This one takes it when the plan is made of exactly the parts the kernel restates
(token embedding, pre-norm blocks of RMSNorm / rotary GQA attention / RMSNorm / SwiGLU,
final RMSNorm, output head; any schedule, windows, biases, shared caches) and the step is a
bfloat16 decode step that fits; everything else runs part by part as before.  The plan
builder of the architecture attaches it (``models/dense_decoder.py``); no part knows of it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Dict, List, Optional

import torch

from ..csrc import ops
from ..csrc.build import load_library
from ..parts import (GQAAttention, ModelPlan, NormedHead, OutputHead, PreNormBlock, RMSNorm,
                     SwiGLU, TokenEmbedding)

MAX_TOKENS = 8
MAX_GROUPS = 4
_TICKETS = 512          # (token, KV head) pairs of a step


class _Layer(ctypes.Structure):
    _fields_ = [("w_qkv", c_void_p), ("b_qkv", c_void_p), ("w_o", c_void_p), ("w_gate_up", c_void_p),
                ("w_down", c_void_p), ("norm_attn", c_void_p), ("norm_ffn", c_void_p),
                ("k_pages", c_void_p), ("v_pages", c_void_p), ("eps_attn", c_float), ("eps_ffn", c_float),
                ("group", c_int), ("window", c_int), ("write_cache", c_int), ("pad", c_int)]


class _Params(ctypes.Structure):
    _fields_ = [("layers", c_void_p), ("layer_begin", c_int), ("layer_end", c_int), ("run_head", c_int),
                ("T", c_int), ("H", c_int), ("I", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int),
                ("V", c_int), ("page_size", c_int), ("scale_log2", c_float), ("positions", c_void_p),
                ("block_tables", c_void_p * MAX_GROUPS), ("bt_stride", c_int * MAX_GROUPS),
                ("cos_tab", c_void_p), ("sin_tab", c_void_p), ("residual", c_void_p), ("qkv", c_void_p),
                ("attn_out", c_void_p), ("hmid", c_void_p), ("part_o", c_void_p), ("part_ml", c_void_p),
                ("tickets", c_void_p), ("splits", c_int), ("final_norm", c_void_p), ("final_eps", c_float),
                ("head_w", c_void_p), ("logits", c_void_p), ("barrier", c_void_p), ("error", c_void_p)]


#: turn the fused decode step off (every step then runs part by part)
ENABLED = True
#: ... for models whose residual stream is wider than this (0: no limit)
MAX_WIDTH = 0

_LOG2E = 1.4426950408889634


class DenseDecodeStep:
    """Built once per plan; ``run`` returns the step's logits, or NotImplemented."""

    def __init__(self, plan: ModelPlan) -> None:
        self.plan = plan
        self.ok = self._plan_fits(plan)
        self._per_cache: Dict[int, dict] = {}
        self._lib = None
        self.steps_run = 0

    # ------------------------------------------------------------------ what the kernel restates
    @staticmethod
    def _plan_fits(plan: ModelPlan) -> bool:
        if type(plan.embedding) is not TokenEmbedding or type(plan.output) is not NormedHead:
            return False
        if type(plan.output.norm) is not RMSNorm or type(plan.output.head) is not OutputHead:
            return False
        if not plan.layers:
            return False
        first = None
        for block in plan.layers:
            if type(block) is not PreNormBlock:
                return False
            a, f = block.mixer, block.ffn
            if type(block.mixer_norm) is not RMSNorm or type(block.ffn_norm) is not RMSNorm \
                    or type(a) is not GQAAttention or type(f) is not SwiGLU:
                return False
            if not a.rotary:
                return False
            sig = (a.width, a.num_heads, a.num_kv_heads, a.head_dim, a.scale, f.inner,
                   id(a.position) if a.position is not None else id(plan.position))
            first = first or sig
            if sig != first:
                return False
        a = plan.layers[0].mixer
        group = a.num_heads // a.num_kv_heads
        return (a.head_dim % 16 == 0 and a.head_dim <= 128 and group <= 8 and a.width % 8 == 0
                and plan.layers[0].ffn.inner % 8 == 0 and (a.num_heads * a.head_dim) % 8 == 0)

    def _library(self):
        if self._lib is None:
            lib = load_library("decode_step")
            if lib.hb_decode_step_layer_bytes() != ctypes.sizeof(_Layer) or \
                    lib.hb_decode_step_param_bytes() != ctypes.sizeof(_Params):
                raise ops.KernelError("decode_step: the parameter layout of the library and of the "
                                      "Python side differ")
            lib.hb_decode_step.argtypes = [c_void_p, c_void_p]
            lib.hb_decode_step.restype = c_int
            self._lib = lib
        return self._lib

    # ------------------------------------------------------------------ per cache: the layer table
    def _for_cache(self, cache, device) -> dict:
        hit = self._per_cache.get(id(cache))
        if hit is not None and hit["cache"] is cache:
            return hit
        plan = self.plan
        rows = (_Layer * len(plan.schedule))()
        for entry, run in enumerate(plan.schedule):
            block = plan.layers[run.layer]
            a, f = block.mixer, block.ffn
            view = cache.layer_cache(entry)
            rows[entry] = _Layer(
                a.w_qkv.data_ptr(), a.b_qkv.data_ptr() if a.b_qkv is not None else 0, a.w_o.data_ptr(),
                f.w_gate_up.data_ptr(), f.w_down.data_ptr(), block.mixer_norm.weight.data_ptr(),
                block.ffn_norm.weight.data_ptr(), view.k_pages.data_ptr(), view.v_pages.data_ptr(),
                block.mixer_norm.eps, block.ffn_norm.eps, view.group, int(a.window or 0),
                1 if view.write else 0, 0)
        table = torch.frombuffer(bytearray(bytes(rows)), dtype=torch.uint8).to(device)
        hit = {"cache": cache, "layers": table,
               "tickets": torch.zeros(_TICKETS, dtype=torch.int32, device=device),
               "barrier": torch.zeros(4, dtype=torch.int32, device=device),
               "error": torch.zeros(1, dtype=torch.int32, device=device)}
        self._per_cache[id(cache)] = hit
        _error_words.append((hit["error"], hit["tickets"]))
        return hit

    # ------------------------------------------------------------------ the step
    def fits(self, ctx, cache) -> bool:
        plan = self.plan
        a = plan.layers[0].mixer
        if not (ENABLED and self.ok and ctx.act_dtype == torch.bfloat16 and ctx.decode_only
                and 0 < ctx.num_tokens <= MAX_TOKENS and ctx.num_wanted == ctx.num_tokens
                and ctx.num_seqs == ctx.num_tokens and len(cache.groups) <= MAX_GROUPS):
            return False
        if MAX_WIDTH and a.width > MAX_WIDTH:
            return False
        if a.num_kv_heads * ctx.num_tokens > _TICKETS:
            return False
        return all(cache.layer_cache(e) is not None for e in range(len(plan.schedule)))

    def run(self, ctx, cache):
        if not self.fits(ctx, cache):
            return NotImplemented
        plan = self.plan
        a, f = plan.layers[0].mixer, plan.layers[0].ffn
        dev = ctx.device
        state = self._for_cache(cache, dev)
        lib = self._library()
        if plan.position is not None:
            plan.position.prepare(ctx)
        cos, sin = a._rotary_tables(ctx)
        if cos is None or cos.shape[1] * 2 != a.head_dim:
            return NotImplemented
        T, H, I = ctx.num_tokens, a.width, f.inner
        nh, nkv, hd = a.num_heads, a.num_kv_heads, a.head_dim
        V = plan.output.head.vocab
        residual = plan.embedding.forward(ctx)
        sms = ops.sm_count(dev)
        most = max(1, min(32, ctx.max_context_len // 256))
        splits = max(1, min(most, sms // (T * nkv)))
        bf = torch.bfloat16
        qkv = torch.empty((T, (nh + 2 * nkv) * hd), dtype=bf, device=dev)
        attn_out = torch.empty((T, nh * hd), dtype=bf, device=dev)
        hmid = torch.empty((T, I), dtype=bf, device=dev)
        part_o = torch.empty((T * nh * splits * hd,), dtype=torch.float32, device=dev) if splits > 1 else None
        part_ml = torch.empty((T * nh * splits * 2,), dtype=torch.float32, device=dev) if splits > 1 else None
        logits = torch.empty((T, V), dtype=torch.float32, device=dev)
        state["barrier"].zero_()
        p = _Params()
        p.layers = state["layers"].data_ptr()
        p.layer_begin, p.layer_end, p.run_head = 0, len(plan.schedule), 1
        p.T, p.H, p.I, p.nh, p.nkv, p.hd, p.V, p.page_size = T, H, I, nh, nkv, hd, V, cache.page_size
        p.scale_log2 = a.scale * _LOG2E
        p.positions = ctx.positions.data_ptr()
        for g, table in enumerate(ctx.block_tables):
            p.block_tables[g] = table.data_ptr()
            p.bt_stride[g] = table.shape[1]
        p.cos_tab, p.sin_tab = cos.data_ptr(), sin.data_ptr()
        p.residual, p.qkv, p.attn_out, p.hmid = (residual.data_ptr(), qkv.data_ptr(), attn_out.data_ptr(),
                                                 hmid.data_ptr())
        p.part_o = part_o.data_ptr() if part_o is not None else 0
        p.part_ml = part_ml.data_ptr() if part_ml is not None else 0
        p.tickets = state["tickets"].data_ptr()
        p.splits = splits
        p.final_norm = plan.output.norm.weight.data_ptr()
        p.final_eps = plan.output.norm.eps
        p.head_w = plan.output.head.weight.data_ptr()
        p.logits = logits.data_ptr()
        p.barrier = state["barrier"].data_ptr()
        p.error = state["error"].data_ptr()
        status = lib.hb_decode_step(ctypes.addressof(p), ops._stream())
        ops.launch_count += 1
        if status != 0:
            raise ops.KernelError(f"decode_step: status {status}")
        self.steps_run += 1
        return logits


_error_words: List[tuple] = []


def check_errors() -> None:
    """Raise if a fused decode step gave up a bounded wait (synchronises)."""
    for word, tickets in _error_words:
        code = int(word.item())
        if code:
            word.zero_()
            tickets.zero_()
            raise ops.KernelError(f"decode_step: a block gave up waiting at the barrier between two phases "
                                  f"(code {code}); the results of that step are not valid")
