"""Python faces of the CUDA launchers: argument checks, then one ctypes call on torch's
current stream. Tensors must live on a CUDA device; a CPU tensor or a missing extension is
an error, never a detour through library code."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from ..errors import KernelError
from . import build

PAGE = 64                      # tokens of a cache page; CML_PAGE in common.cuh
F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}
EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU = 0, 1, 2, 3

_ERRORS = {-2: "unsupported element type", -3: "a size is outside what the kernel takes",
           -4: "a pointer or stride is not aligned as the kernel needs"}

_SIGNATURES = {
    ("rowwise", "cml_embed_gather"): [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    ("rowwise", "cml_embed_positions"): [c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_void_p, c_void_p],
    ("rowwise", "cml_rmsnorm"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p,
                                 c_int, c_long, c_void_p],
    ("rowwise", "cml_add_partials"): [c_void_p, c_void_p, c_int, c_long, c_void_p],
    ("rowwise", "cml_swiglu_packed"): [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("rope_kv", "cml_rope_kv_write"): [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ("rope_kv", "cml_rope_kv_from_partials"): [c_void_p, c_int, c_long, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                               c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                               c_int, c_int, c_int, c_void_p],
    ("gemm_tc", "cml_gemm_tc"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long, c_int, c_int,
                                 c_int, c_void_p, c_void_p],
    ("gemm_tc", "cml_gemm_tc_pair"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long, c_int,
                                      c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    ("gemm_tc", "cml_gemm_tc_pair_partial"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long,
                                              c_long, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    ("gemm_tc", "cml_gemm_tc_pair_add_norm"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long,
                                               c_void_p, c_void_p, c_int, c_void_p, c_long, c_void_p, c_void_p],
    ("rowwise", "cml_scale_rows"): [c_void_p, c_int, c_long, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
    ("attention_simt", "cml_attn_paged_simt"): [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                c_void_p, c_void_p],
    ("attention_simt", "cml_attn_simt_smem_bytes"): [c_int, c_int, c_int, c_int],
    ("attention_mma", "cml_attn_paged_mma"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                              c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                              c_void_p, c_void_p],
    ("attention_mma", "cml_attn_decode_fused"): [c_void_p, c_int, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_float, c_int, c_void_p, c_int, c_void_p],
    ("attention_tc", "cml_attn_prefill_tc"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long, c_void_p,
                                              c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    ("attention_tc", "cml_attn_prefill_tc_ext"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long, c_void_p,
                                                  c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                                  c_int, c_void_p, c_void_p, c_long, c_int, c_void_p, c_void_p],
    ("attention_tc", "cml_attn_prefill_tc_maps"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long, c_void_p,
                                                   c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                                   c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_float, c_int, c_int,
                                                   c_void_p, c_void_p],
    ("attention_window", "cml_maps_difference"): [c_void_p, c_long, c_void_p, c_long, c_int, c_long, c_int, c_int, c_float, c_float,
                                                  c_float, c_void_p],
    ("attention_tc", "cml_attn_prefill_tc_penalty"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long, c_void_p,
                                                      c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                      c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                                      c_void_p, c_void_p],
    ("gemm_simt", "cml_gemm_tn_simt"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p, c_void_p, c_void_p],
    ("gemm_simt", "cml_gemv_f32_scratch_bytes"): [c_int, c_int, c_int, c_int],
    ("gemm_simt", "cml_gemv_f32_partial_splits"): [c_int, c_int, c_int, c_int, c_int],
    ("gemm_simt", "cml_gemv_f32_partial"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_long, c_int, c_int,
                                            c_int, c_int, c_void_p, c_void_p],
    ("sampling", "cml_argmax_rows"): [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "cml_adjust_dense"): [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "cml_count_tokens"): [c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("sampling", "cml_adjust_logits"): [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_float,
                                        c_void_p],
    ("sampling", "cml_decode_loop_size"): [],
    ("sampling", "cml_decode_loop_init"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "cml_decode_loop_run"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                         c_int, c_float, c_int, c_float, c_float, ctypes.c_ulonglong, c_void_p, c_void_p],
    ("sampling", "cml_decode_fed_run"): [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    ("sampling", "cml_draws_at"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    ("sampling", "cml_sample_rows"): [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_float, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p],
    ("token_ops", "cml_bigram_embed"): [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, ctypes.c_longlong, ctypes.c_longlong,
                                        ctypes.c_longlong, c_void_p, c_void_p],
    ("token_ops", "cml_keep_last_rows"): [c_void_p, c_int, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_void_p],
    ("token_ops", "cml_token_shift"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int, c_int, c_void_p],
    ("token_ops", "cml_rmsnorm_shift"): [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int, c_int, c_int, c_float, c_void_p, c_int, c_long, c_void_p],
    ("token_ops", "cml_add_rows_vec"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    ("token_ops", "cml_gelu_tanh"): [c_void_p, c_int, c_long, c_void_p],
    ("token_ops", "cml_act_from_partials"): [c_void_p, c_int, c_long, c_void_p, c_int, c_long, c_int, c_void_p, c_int, c_void_p],
    ("token_ops", "cml_bias_act"): [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    ("token_ops", "cml_gate_rows"): [c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_int, c_void_p],
    ("token_ops", "cml_softcap"): [c_void_p, c_long, c_float, c_void_p],
    ("token_ops", "cml_post_norm_add"): [c_void_p, c_int, c_long, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_void_p,
                                         c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    ("token_ops", "cml_sum_norm"): [c_void_p, c_int, c_long, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_void_p, c_int,
                                    c_int, c_int, c_void_p],
    ("token_ops", "cml_gelu_mul_lookup"): [c_void_p, c_long, c_int, c_long, c_void_p, c_int, c_long, c_int, c_void_p, c_int,
                                           c_void_p, c_int, c_int, c_void_p],
    ("token_ops", "cml_cast_rows"): [c_void_p, c_void_p, c_int, c_long, c_void_p],
    ("token_ops", "cml_norm_combine"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                        c_float, c_float, c_void_p],
    ("recurrence", "cml_conv_unit"): [c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_long, c_void_p, c_void_p,
                                      c_void_p, c_int, c_void_p],
    ("recurrence", "cml_delta_scan"): [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_long, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_int, c_void_p],
    ("recurrence", "cml_memory_scan"): [c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                        c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_int, c_void_p],
    ("recurrence", "cml_head_norm_gate"): [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_long, c_int, c_void_p, c_int,
                                           c_int, c_int, c_int, c_float, c_int, c_void_p],
    ("attention_window", "cml_qk_norm_kv_write"): [c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p,
                                                   c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_int, c_int, c_int, c_void_p],
    ("attention_window", "cml_window_attention"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_int, c_int, c_int,
                                                   c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_int, c_float, c_float,
                                                   c_float, c_float, c_int, c_int, c_void_p],
    ("attention_window", "cml_qkv_prepare"): [c_void_p, c_long, c_int, c_long, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                              c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p],
    ("attention_latent", "cml_latent_prepare"): [c_void_p, c_long, c_int, c_long, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p,
                                                 c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                 c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ("attention_latent", "cml_head_product"): [c_void_p, c_long, c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int,
                                               c_int, c_void_p],
    ("attention_latent", "cml_latent_prompt"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int,
                                                c_int, c_float, c_void_p, c_int, c_int, c_long, c_void_p],
    ("recurrence", "cml_retention_scan"): [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("recurrence", "cml_rotate_rows"): [c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p,
                                        c_int, c_float, c_void_p],
    ("token_ops", "cml_scale_values"): [c_void_p, c_long, c_float, c_void_p],
    ("experts", "cml_route_topk"): [c_void_p, c_long, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                    c_float, c_void_p, c_void_p, c_void_p],
    ("experts", "cml_expert_plan"): [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    ("gemm_tc", "cml_gemm_tc_grouped"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_long, c_int,
                                         c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("experts", "cml_expert_gather"): [c_void_p, c_int, c_long, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                       c_int, c_int, c_void_p, c_void_p, c_void_p],
    ("experts", "cml_expert_gemm"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p],
    ("experts", "cml_expert_combine"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_long, c_void_p, c_int,
                                        c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    ("random_fill", "cml_random_fill"): [c_void_p, c_int, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_ulonglong,
                                         ctypes.c_double, ctypes.c_double, c_void_p],
}
_fns: dict = {}
_libs: dict = {}
_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process (graph replays included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _fn(module: str, name: str):
    f = _fns.get(name)
    if f is None:
        lib = build.load(module)
        if module not in _libs:
            _libs[module] = lib
            _apply_dependent_launch(lib)
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[(module, name)]
        f.restype = c_int
        _fns[name] = f
    return f


def _check(code: int, what: str, launches: int = 1):
    global _launches
    _launches += launches
    if code != 0:
        if code in _ERRORS:
            raise KernelError(f"{what}: {_ERRORS[code]}")
        raise KernelError(f"{what}: CUDA error {code} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _dev(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("camelid_b200 kernels run on CUDA tensors only; there is no CPU path")


def _p(t):
    return None if t is None else t.data_ptr()


_sm_counts: dict = {}


def sm_count(device) -> int:
    """Multiprocessors of ``device`` (the number the launchers read from the runtime too)."""
    device = torch.device(device)
    n = _sm_counts.get(device)
    if n is None:
        n = int(torch.cuda.get_device_properties(device).multi_processor_count)
        _sm_counts[device] = n
    return n


_dependent_launch = True


def set_dependent_launch(on: bool) -> None:
    """Whether kernels are launched with programmatic dependent launch (the default). Applies
    to every kernel module, those loaded later included."""
    global _dependent_launch
    if bool(on) == _dependent_launch:
        return
    _dependent_launch = bool(on)
    for lib in _libs.values():
        _apply_dependent_launch(lib)


class GateAct(tuple):
    """(alpha, limit, shift) of a gated feed-forward's activation: with g' = min(g, limit) and u' = clamp(u, -limit,
    limit), out = g' * sigmoid(alpha * g') * (u' + shift). ``SILU_GATE`` (1, inf, 0) is SwiGLU."""
    def __new__(cls, alpha: float = 1.0, limit: float = float("inf"), shift: float = 0.0):
        return super().__new__(cls, (float(alpha), float(limit), float(shift)))


SILU_GATE = GateAct()
_gate_act_set: dict = {}


def _gate_act(module: str, act) -> None:
    """Tell ``module`` which activation its gated epilogues apply from now on; the launchers hand the numbers to their
    kernels by value, so every wrapper of a gated product calls this right before its launch."""
    act = SILU_GATE if act is None else act
    if _gate_act_set.get(module) == act:
        return
    _fn(module, next(n for m, n in _SIGNATURES if m == module))          # make sure the module is loaded
    setter = _libs[module].cml_set_gate_act
    setter.argtypes, setter.restype = [c_float, c_float, c_float], None
    setter(*act)
    _gate_act_set[module] = act


def _apply_dependent_launch(lib) -> None:
    try:
        setter = lib.cml_set_dependent_launch
    except AttributeError:          # a module without kernels that depend on their predecessors
        return
    setter.argtypes, setter.restype = [c_int], None
    setter(1 if _dependent_launch else 0)


try:        # the raw handle of the current stream without building a Stream object (a third of a launch's host time)
    _raw_stream, _device_now = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:      # a torch without these: the public way
    _raw_stream = None


def _stream():
    if _raw_stream is not None:
        return _raw_stream(_device_now())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"element type {dt} is not supported (float32 and bfloat16 are)") from None


# ---------------------------------------------------------------------------------------

def random_fill(out: torch.Tensor, key: int, first: int, mean: float, std: float):
    """out.view(-1)[i] = element ``first + i`` of the counter-based generator under ``key``
    (weights/counter_random.py is the host's definition of the same numbers)."""
    _dev(out)
    assert out.is_contiguous()
    _check(_fn("random_fill", "cml_random_fill")(_p(out), dtype_code(out.dtype), out.numel(), int(key), int(first),
                                                 float(mean), float(std), _stream()), "random_fill")


def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, err: torch.Tensor):
    """out[r] = table[tokens[r]] as float32. ``err`` (int32[1]) gets bit 1 on a bad id."""
    _dev(table, tokens, out, err)
    rows, hidden = out.shape
    assert table.shape[1] == hidden and tokens.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous() and tokens.numel() >= rows
    _check(_fn("rowwise", "cml_embed_gather")(_p(table), dtype_code(table.dtype), _p(tokens), _p(out), rows, hidden,
                                             table.shape[0], _p(err), _stream()), "embed_gather")


def embed_positions(table: torch.Tensor, tokens: torch.Tensor, scale: float, positions, row_pos, out: torch.Tensor, err: torch.Tensor,
                    x_out=None):
    """out[r] = scale * table[tokens[r]] + positions[row_pos[r]] as float32 (``positions`` None: no second term);
    ``x_out``: the same rows in the table's type. ``err`` gets bit 1 on a bad id, bit 2 on a position beyond the table."""
    _dev(table, tokens, positions, row_pos, out, err, x_out)
    rows, hidden = out.shape
    assert table.shape[1] == hidden and tokens.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous() and tokens.numel() >= rows
    if positions is not None:
        assert positions.dtype == table.dtype and positions.shape[1] == hidden and positions.is_contiguous()
        assert row_pos.dtype == torch.int32 and row_pos.numel() >= rows
    if x_out is not None:
        assert x_out.dtype == table.dtype and x_out.shape == out.shape and x_out.is_contiguous()
    _check(_fn("rowwise", "cml_embed_positions")(_p(table), dtype_code(table.dtype), _p(tokens), float(scale), _p(positions), _p(row_pos),
                                                positions.shape[0] if positions is not None else 0, _p(out), _p(x_out), rows, hidden,
                                                table.shape[0], _p(err), _stream()), "embed_positions")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, rows_index: torch.Tensor | None = None,
            partial: torch.Tensor | None = None):
    """out[r] = rmsnorm(x[rows_index[r] or r]) * weight; x float32, out float32 or bfloat16.
    ``partial`` (float32 [splits, x rows, hidden]) is first added to x, split by split; without
    ``rows_index`` the sum is written back to x."""
    _dev(x, weight, out, rows_index, partial)
    rows, hidden = out.shape
    assert x.dtype == torch.float32 and x.shape[1] == hidden and weight.shape[0] == hidden
    assert x.is_contiguous() and out.is_contiguous()
    if rows_index is not None:
        assert rows_index.dtype == torch.int32 and rows_index.numel() >= rows
    n_splits, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1:] == x.shape
        n_splits, stride = partial.shape[0], partial.stride(0)
    _check(_fn("rowwise", "cml_rmsnorm")(_p(x), _p(weight), dtype_code(weight.dtype), _p(out), dtype_code(out.dtype),
                                        _p(rows_index), rows, hidden, float(eps), _p(partial), n_splits, stride,
                                        _stream()), "rmsnorm")


def add_partials(x: torch.Tensor, partial: torch.Tensor):
    """x += sum over splits of partial[split] (float32), splits in index order."""
    _dev(x, partial)
    assert x.dtype == torch.float32 and partial.dtype == torch.float32 and partial.shape[1:] == x.shape
    assert x.is_contiguous() and partial.is_contiguous()
    _check(_fn("rowwise", "cml_add_partials")(_p(x), _p(partial), partial.shape[0], x.numel(), _stream()), "add_partials")


def swiglu_packed(gu: torch.Tensor, act: torch.Tensor, group: int):
    _dev(gu, act)
    rows, inter = act.shape
    assert gu.shape == (rows, 2 * inter) and gu.dtype == act.dtype and gu.is_contiguous() and act.is_contiguous()
    _check(_fn("rowwise", "cml_swiglu_packed")(_p(gu), _p(act), dtype_code(act.dtype), rows, inter, group, _stream()),
           "swiglu_packed")


def rope_kv_write(qkv: torch.Tensor, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq, rotary_dim: int,
                  n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool):
    """Rotate q (and k) of packed rows in place; write k and v into their cache pages."""
    _dev(qkv, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq)
    rows = qkv.shape[0]
    assert qkv.stride(1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rotary_dim
    need = (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    assert qkv.shape[1] >= need, (qkv.shape, need)
    if write_kv:
        assert k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype
        assert k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
        max_blocks = block_table.shape[1]
    else:
        max_blocks = 0
    _check(_fn("rope_kv", "cml_rope_kv_write")(
        _p(qkv), dtype_code(qkv.dtype), rows, qkv.stride(0), _p(row_pos), _p(row_seq), _p(block_table), max_blocks,
        _p(k_pages), _p(v_pages), _p(inv_freq), rotary_dim, n_heads, n_kv_heads, head_dim, 1 if write_kv else 0,
        _stream()), "rope_kv_write")


def rope_kv_from_partials(partial: torch.Tensor, q_out: torch.Tensor, row_pos, row_seq, block_table, k_pages, v_pages,
                          inv_freq, rotary_dim: int, n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool):
    """The same as rope_kv_write on the split sums ``partial`` (float32 [splits, rows, width]) of
    the q/k/v product; the rotated q goes to ``q_out`` in the compute type."""
    _dev(partial, q_out, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq)
    n_splits, rows, width = partial.shape
    assert partial.dtype == torch.float32 and partial.is_contiguous() and q_out.stride(1) == 1
    assert q_out.shape == (rows, n_heads * head_dim) and inv_freq.numel() * 2 == rotary_dim
    if write_kv:
        assert k_pages.dtype == q_out.dtype and k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim)
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
    _check(_fn("rope_kv", "cml_rope_kv_from_partials")(
        _p(partial), n_splits, partial.stride(0), width, _p(q_out), q_out.stride(0), dtype_code(q_out.dtype), rows,
        _p(row_pos), _p(row_seq), _p(block_table), block_table.shape[1] if write_kv else 0, _p(k_pages), _p(v_pages),
        _p(inv_freq), rotary_dim, n_heads, n_kv_heads, head_dim, 1 if write_kv else 0, _stream()),
        "rope_kv_from_partials")


# ---------------------------------------------------------------------------------------
# what a sequence carries from token to token besides keys and values, and small row-wise steps

def bigram_embed(table: torch.Tensor, bigram, tokens, row_seq, row_pos, seq_row0, seq_new, seq_slot, prev_state, out,
                 n_seqs: int, buckets: int, mul_prev: int, mul_cur: int, err: torch.Tensor):
    """out[r] = table[tokens[r]] (+ bigram[hash of the previous and this token], the last row for a
    sequence's first token) as float32; ``prev_state`` (int32 [slots]) gives the token before a
    step's first row and takes the step's last token."""
    _dev(table, bigram, tokens, row_seq, row_pos, seq_row0, seq_new, seq_slot, prev_state, out, err)
    rows, hidden = out.shape
    assert table.shape[1] == hidden and tokens.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous()
    if bigram is not None:
        assert bigram.dtype == table.dtype and bigram.shape == (buckets + 1, hidden) and bigram.is_contiguous()
        assert prev_state.dtype == torch.int32 and prev_state.is_contiguous()
    _check(_fn("token_ops", "cml_bigram_embed")(_p(table), _p(bigram), dtype_code(table.dtype), _p(tokens), _p(row_seq),
                                                _p(row_pos), _p(seq_row0), _p(seq_new), _p(seq_slot), _p(prev_state), _p(out),
                                                rows, n_seqs, hidden, table.shape[0], int(buckets or 1), int(mul_prev or 0),
                                                int(mul_cur or 0), _p(err), _stream()),
           "bigram_embed", 2 if bigram is not None else 1)


def keep_last_rows(src: torch.Tensor, col0: int, width: int, state: torch.Tensor, seq_row0, seq_new, seq_start, seq_slot,
                   n_seqs: int):
    """state[slot] (float32 [slots, keep, width]) = columns col0.. of each sequence's last ``keep`` rows
    after this step (rows of ``src`` where the step brought them, else what the state held)."""
    _dev(src, state, seq_row0, seq_new, seq_start, seq_slot)
    assert src.dim() == 2 and src.stride(1) == 1 and col0 + width <= src.shape[1]
    assert state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 3 and state.shape[2] == width
    _check(_fn("token_ops", "cml_keep_last_rows")(_p(src), dtype_code(src.dtype), src.stride(0), col0, width, state.shape[1],
                                                  _p(seq_row0), _p(seq_new), _p(seq_start), _p(seq_slot), _p(state), n_seqs,
                                                  _stream()), "keep_last_rows")


def token_shift(h: torch.Tensor, mix: torch.Tensor, state: torch.Tensor, row_seq, row_pos, seq_row0, seq_slot,
                out: torch.Tensor):
    """out[r] = h[r] + (h[r - 1] - h[r]) * mix within a sequence; zeros before the first token,
    ``state[slot]`` (float32 [slots, hidden]) before a step's first row."""
    _dev(h, mix, state, row_seq, row_pos, seq_row0, seq_slot, out)
    rows, hidden = h.shape
    assert h.is_contiguous() and out.is_contiguous() and out.shape == h.shape and out.dtype == h.dtype
    assert mix.numel() == hidden and state.dtype == torch.float32 and state.shape[-1] == hidden and state.is_contiguous()
    _check(_fn("token_ops", "cml_token_shift")(_p(h), dtype_code(h.dtype), _p(mix), dtype_code(mix.dtype), _p(state),
                                               _p(row_seq), _p(row_pos), _p(seq_row0), _p(seq_slot), _p(out), rows, hidden,
                                               _stream()), "token_shift")


def rmsnorm_shift(x: torch.Tensor, weight: torch.Tensor, eps: float, mix: torch.Tensor, state: torch.Tensor, row_seq, row_pos,
                  seq_slot, out: torch.Tensor, partial: torch.Tensor | None = None):
    """One-token steps: ``rmsnorm`` (with the pending split sums added and written back), ``token_shift`` and
    the keeping of the normed row in one launch; every row is the one new row of its sequence."""
    _dev(x, weight, mix, state, row_seq, row_pos, seq_slot, out, partial)
    rows, hidden = out.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (rows, hidden) and out.is_contiguous()
    assert mix.dtype == torch.float32 and mix.numel() == hidden and weight.numel() == hidden
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[-1] == hidden
    n_splits, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1:] == x.shape
        n_splits, stride = partial.shape[0], partial.stride(0)
    _check(_fn("token_ops", "cml_rmsnorm_shift")(_p(x), _p(weight), dtype_code(weight.dtype), _p(mix), _p(state), _p(row_seq),
                                                 _p(row_pos), _p(seq_slot), _p(out), dtype_code(out.dtype), rows, hidden,
                                                 float(eps), _p(partial), n_splits, stride, _stream()), "rmsnorm_shift")


def add_rows_vec(h: torch.Tensor, base, vec: torch.Tensor):
    """h[r] += (base[r] if given) + vec, float32 rows in place."""
    _dev(h, base, vec)
    rows, hidden = h.shape
    assert h.dtype == torch.float32 and h.is_contiguous() and vec.numel() == hidden and vec.is_contiguous()
    if base is not None:
        assert base.dtype == torch.float32 and base.shape == h.shape and base.is_contiguous()
    _check(_fn("token_ops", "cml_add_rows_vec")(_p(h), _p(base), _p(vec), dtype_code(vec.dtype), rows, hidden, _stream()),
           "add_rows_vec")


def gelu_tanh_(x: torch.Tensor):
    """x = 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))) in place."""
    _dev(x)
    assert x.is_contiguous()
    _check(_fn("token_ops", "cml_gelu_tanh")(_p(x), dtype_code(x.dtype), x.numel(), _stream()), "gelu_tanh")


ACT_NONE, ACT_GELU_TANH, ACT_RELU_SQUARED, ACT_GELU_ERF = 0, 1, 2, 3
ACTIVATIONS = {None: ACT_NONE, "none": ACT_NONE, "gelu_tanh": ACT_GELU_TANH, "relu_squared": ACT_RELU_SQUARED,
               "gelu_erf": ACT_GELU_ERF}


def act_from_partials(part: torch.Tensor, out: torch.Tensor, gelu: bool = False, act: int | None = None, bias=None):
    """out = act(sum over splits of part + bias) in the compute type; part float32 [splits, rows, n]; ``act`` one of
    the ACT_* codes (``gelu``: the tanh form of GELU); ``bias`` float32 [n] or None."""
    _dev(part, out, bias)
    assert part.dtype == torch.float32 and part.dim() == 3 and part.is_contiguous() and out.is_contiguous()
    assert tuple(out.shape) == tuple(part.shape[1:])
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == out.shape[-1] and bias.is_contiguous())
    code = act if act is not None else (ACT_GELU_TANH if gelu else ACT_NONE)
    _check(_fn("token_ops", "cml_act_from_partials")(_p(part), part.shape[0], part.stride(0), _p(out), dtype_code(out.dtype),
                                                     out.numel(), code, _p(bias), out.shape[-1], _stream()), "act_from_partials")


def bias_act_(x: torch.Tensor, bias, act: int):
    """x[r, c] = act(x[r, c] + bias[c]) in place; ``bias`` float32 [columns] or None; ``act`` one of the ACT_* codes."""
    _dev(x, bias)
    assert x.dim() == 2 and x.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == x.shape[1] and bias.is_contiguous())
    _check(_fn("token_ops", "cml_bias_act")(_p(x), dtype_code(x.dtype), _p(bias), x.shape[0], x.shape[1], int(act), _stream()),
           "bias_act")


def gate_rows_(x: torch.Tensor, gate: torch.Tensor, gate_col: int):
    """x[r, c] *= sigmoid(gate[r, gate_col + c]) in place; gate float32."""
    _dev(x, gate)
    rows, width = x.shape
    assert x.is_contiguous() and gate.dtype == torch.float32 and gate.stride(1) == 1 and gate_col + width <= gate.shape[1]
    _check(_fn("token_ops", "cml_gate_rows")(_p(x), dtype_code(x.dtype), _p(gate), gate.stride(0), gate_col, rows, width,
                                             _stream()), "gate_rows")


def softcap_(x: torch.Tensor, cap: float):
    """x = cap * tanh(x / cap) in place (float32)."""
    _dev(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(_fn("token_ops", "cml_softcap")(_p(x), x.numel(), float(cap), _stream()), "softcap")


def scale_(x: torch.Tensor, factor: float):
    """x *= factor in place (float32)."""
    _dev(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(_fn("token_ops", "cml_scale_values")(_p(x), x.numel(), float(factor), _stream()), "scale_values")


def norm_combine(branches: list, residual: torch.Tensor, eps: float, coef: float, biases: list | None = None):
    """residual[r] += coef * sum of rmsnorm(y[r] + bias) * w over ``branches`` = [(y, w)], y float32
    [rows, hidden] or [splits, rows, hidden] (splits summed first), w [hidden]; ``biases``: per branch a
    float32 [hidden] vector or None."""
    rows, hidden = residual.shape
    assert 1 <= len(branches) <= 4 and residual.dtype == torch.float32 and residual.is_contiguous()
    n = len(branches)
    ys, ws, bs, splits, strides = (c_void_p * n)(), (c_void_p * n)(), (c_void_p * n)(), (c_int * n)(), (c_long * n)()
    for i, b in enumerate(biases or [None] * n):
        if b is not None:
            _dev(b)
            assert b.dtype == torch.float32 and b.numel() == hidden and b.is_contiguous()
        bs[i] = _p(b)
    for i, (y, w) in enumerate(branches):
        _dev(y, w)
        if y.dim() == 2:
            y = y.unsqueeze(0)
        assert y.dtype == torch.float32 and y.shape[1:] == (rows, hidden) and y.stride(2) == 1 and y.stride(1) == hidden
        assert w.numel() == hidden and w.is_contiguous() and w.dtype == branches[0][1].dtype
        ys[i], ws[i], splits[i], strides[i] = y.data_ptr(), w.data_ptr(), y.shape[0], y.stride(0)
    _check(_fn("token_ops", "cml_norm_combine")(ys, ws, bs, splits, strides, n, dtype_code(branches[0][1].dtype), _p(residual),
                                                rows, hidden, float(eps), float(coef), _stream()), "norm_combine")


def post_norm_add(y: torch.Tensor, bias, w_post: torch.Tensor, eps: float, coef: float, residual: torch.Tensor,
                  w_next=None, eps_next: float = 0.0, x_out=None):
    """residual[r] += coef * rmsnorm(y[r] + bias) * w_post, and with ``x_out`` also x_out[r] = rmsnorm(residual[r]) * w_next
    (the norm before the next sublayer) in the same pass. y float32 [rows, hidden] or split sums [splits, rows, hidden]."""
    _dev(y, bias, w_post, residual, w_next, x_out)
    rows, hidden = residual.shape
    if y.dim() == 2:
        y = y.unsqueeze(0)
    assert residual.dtype == torch.float32 and residual.is_contiguous()
    assert y.dtype == torch.float32 and y.shape[1:] == (rows, hidden) and y.stride(2) == 1 and y.stride(1) == hidden
    assert w_post.numel() == hidden and w_post.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == hidden and bias.is_contiguous())
    if x_out is not None:           # without w_next: the stream's rows themselves in x_out's type
        assert w_next is None or (w_next.dtype == w_post.dtype and w_next.numel() == hidden and w_next.is_contiguous())
        assert x_out.shape == (rows, hidden) and x_out.is_contiguous()
    _check(_fn("token_ops", "cml_post_norm_add")(
        _p(y), y.shape[0], y.stride(0), _p(bias), _p(w_post), dtype_code(w_post.dtype), float(eps), float(coef), _p(residual),
        _p(w_next), float(eps_next), _p(x_out), dtype_code(x_out.dtype) if x_out is not None else 0, rows, hidden, _stream()),
        "post_norm_add")


def sum_norm(y: torch.Tensor, bias, w: torch.Tensor, eps: float, alpha: float, residual: torch.Tensor, x_out=None):
    """residual[r] = rmsnorm(alpha * residual[r] + y[r] + bias) * w, the norm after a residual sum, in place; with ``x_out``
    also the new rows in its type. y float32 [rows, hidden] or split sums [splits, rows, hidden]."""
    _dev(y, bias, w, residual, x_out)
    rows, hidden = residual.shape
    if y.dim() == 2:
        y = y.unsqueeze(0)
    assert residual.dtype == torch.float32 and residual.is_contiguous()
    assert y.dtype == torch.float32 and y.shape[1:] == (rows, hidden) and y.stride(2) == 1 and y.stride(1) == hidden
    assert w.numel() == hidden and w.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == hidden and bias.is_contiguous())
    assert x_out is None or (x_out.shape == (rows, hidden) and x_out.is_contiguous())
    _check(_fn("token_ops", "cml_sum_norm")(
        _p(y), y.shape[0], y.stride(0), _p(bias), _p(w), dtype_code(w.dtype), float(eps), float(alpha), _p(residual), _p(x_out),
        dtype_code(x_out.dtype) if x_out is not None else 0, rows, hidden, _stream()), "sum_norm")


def cast_rows(x: torch.Tensor, out: torch.Tensor):
    """out = x (float32) in out's type."""
    _dev(x, out)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == x.shape
    _check(_fn("token_ops", "cml_cast_rows")(_p(x), _p(out), dtype_code(out.dtype), x.numel(), _stream()), "cast_rows")


def gelu_mul_lookup(z: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor, out: torch.Tensor):
    """out[r, c] = gelu_tanh(z[r, c]) * table[tokens[r], col0 + c] in the table's type; z float32 [rows, dim] or split sums
    [splits, rows, dim] that are added first."""
    _dev(z, table, tokens, out)
    if z.dim() == 2:
        z = z.unsqueeze(0)
    rows, dim = out.shape
    assert z.dtype == torch.float32 and z.shape[1:] == (rows, dim) and z.stride(2) == 1
    assert table.stride(1) == 1 and 0 <= col0 and col0 + dim <= table.shape[1] and out.dtype == table.dtype and out.is_contiguous()
    assert tokens.dtype == torch.int32 and tokens.numel() >= rows
    _check(_fn("token_ops", "cml_gelu_mul_lookup")(_p(z), z.stride(1), z.shape[0], z.stride(0), _p(table), dtype_code(table.dtype),
                                                   table.stride(0), int(col0), _p(tokens), table.shape[0], _p(out), rows, dim, _stream()),
           "gelu_mul_lookup")


# ---------------------------------------------------------------------------------------
# recurrent mixers with a matrix state per head

def conv_unit(proj: torch.Tensor, conv_w: torch.Tensor, state: torch.Tensor, row_seq, row_pos, seq_row0, seq_slot,
              out: torch.Tensor, qk_heads: int, heads: int, key_dim: int, value_dim: int, q_scale: float,
              update_state: bool = False, decay=None):
    """Short causal convolution + SiLU over the q, k, v channels at the start of ``proj``'s columns
    (float32), then unit norm of q and k per head, q times ``q_scale``. ``conv_w`` float32
    [channels, taps]; ``state`` float32 [slots, taps - 1, channels]: the inputs before the step. With
    ``update_state`` (only where every sequence brings exactly one row) the state moves on by that row here;
    otherwise ``keep_last_rows`` does that afterwards. ``decay`` = (inputs float32 [rows, heads * key_dim] view, a_log,
    dt_bias, out float32 [rows, heads * key_dim]): the same launch also makes the delta rule's decays
    exp(-exp(a_log[head]) softplus(x + dt_bias))."""
    _dev(proj, conv_w, state, row_seq, row_pos, seq_row0, seq_slot, out)
    channels, taps = conv_w.shape
    rows = out.shape[0]
    assert channels == 2 * qk_heads * key_dim + heads * value_dim and proj.shape[1] >= channels
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and conv_w.dtype == torch.float32 and conv_w.is_contiguous()
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (rows, channels)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (max(taps - 1, 1), channels)
    d_in = d_alog = d_bias = d_out = None
    decay_dim = key_dim
    if decay is not None:
        d_in, d_alog, d_bias, d_out = decay
        _dev(d_in, d_alog, d_bias, d_out)
        decay_dim = d_bias.numel() // heads              # key_dim: a decay per key channel; 1: one per head
        assert decay_dim in (1, key_dim) and d_bias.numel() == heads * decay_dim
        assert d_in.dtype == torch.float32 and d_in.stride(1) == 1 and d_in.shape == (rows, heads * decay_dim)
        assert d_out.dtype == torch.float32 and d_out.is_contiguous() and d_out.shape == (rows, heads * decay_dim)
        assert d_alog.numel() == heads
    _check(_fn("recurrence", "cml_conv_unit")(_p(proj), proj.stride(0), _p(conv_w), _p(state), 1 if update_state else 0, _p(row_seq), _p(row_pos),
                                              _p(seq_row0), _p(seq_slot), _p(out), rows, qk_heads, heads, key_dim, value_dim,
                                              taps, float(q_scale), _p(d_in), d_in.stride(0) if d_in is not None else 0,
                                              _p(d_alog), _p(d_bias), _p(d_out), decay_dim, _stream()), "conv_unit")


def delta_scan(qkv: torch.Tensor, beta_in: torch.Tensor, beta_col: int, decay_in: torch.Tensor, a_log, dt_bias,
               state: torch.Tensor, seq_row0, seq_new, seq_start, seq_slot, out: torch.Tensor, n_seqs: int, heads: int,
               qk_heads: int, key_dim: int, value_dim: int, decay_ready: bool = False):
    """The gated delta rule over each sequence's new rows; ``state`` float32 [slots, heads, value_dim,
    key_dim] (column by column) is read and replaced; ``out`` float32 [rows, heads * value_dim] = S^T q.
    ``decay_ready``: ``decay_in`` holds the decays themselves (``conv_unit`` made them), not their inputs."""
    _dev(qkv, beta_in, decay_in, a_log, dt_bias, state, seq_row0, seq_new, seq_start, seq_slot, out)
    for t in (qkv, beta_in, decay_in, out, state, a_log, dt_bias):
        assert t.dtype == torch.float32 and t.stride(-1) == 1
    assert state.is_contiguous() and state.shape[1:] == (heads, value_dim, key_dim) and out.is_contiguous()
    decay_dim = decay_in.shape[1] // heads               # key_dim: a decay per key channel; 1: one per head
    assert decay_dim in (1, key_dim) and decay_in.shape[1] == heads * decay_dim and out.shape[1] == heads * value_dim
    _check(_fn("recurrence", "cml_delta_scan")(_p(qkv), qkv.stride(0), _p(beta_in), beta_in.stride(0), beta_col, _p(decay_in),
                                               decay_in.stride(0), _p(a_log), _p(dt_bias), _p(state), _p(seq_row0),
                                               _p(seq_new), _p(seq_start), _p(seq_slot), _p(out), n_seqs, heads, qk_heads,
                                               key_dim, value_dim, 1 if decay_ready else 0, decay_dim, _stream()), "delta_scan")


def memory_scan(proj: torch.Tensor, cols: tuple, i_bias, f_bias, cap: float, q_scale: float, state: torch.Tensor,
                state_m: torch.Tensor, seq_row0, seq_new, seq_start, seq_slot, out: torch.Tensor, n_seqs: int, heads: int,
                key_dim: int, value_dim: int):
    """The matrix memory with exponential gates over each sequence's new rows. ``cols``: columns of
    q, k, v, input gate, forget gate in ``proj`` (float32). ``state`` float32 [slots, heads,
    value_dim + 1, key_dim] (column by column, the last column is n), ``state_m`` float32 [slots, heads,
    value_dim + 1] (the running maximum); ``out`` float32 [rows, heads, value_dim + 2]."""
    _dev(proj, i_bias, f_bias, state, state_m, seq_row0, seq_new, seq_start, seq_slot, out)
    for t in (proj, i_bias, f_bias, state, state_m, out):
        assert t.dtype == torch.float32 and t.stride(-1) == 1
    assert state.is_contiguous() and state.shape[1:] == (heads, value_dim + 1, key_dim)
    assert state_m.is_contiguous() and state_m.shape[1:] == (heads, value_dim + 1)
    assert out.is_contiguous() and out.shape[1:] == (heads, value_dim + 2)
    q_col, k_col, v_col, i_col, f_col = cols
    _check(_fn("recurrence", "cml_memory_scan")(_p(proj), proj.stride(0), q_col, k_col, v_col, i_col, f_col, _p(i_bias),
                                                _p(f_bias), float(cap), float(q_scale), _p(state), _p(state_m), _p(seq_row0), _p(seq_new),
                                                _p(seq_start), _p(seq_slot), _p(out), n_seqs, heads, key_dim, value_dim,
                                                _stream()), "memory_scan")


def head_norm_gate(raw: torch.Tensor, with_den: bool, w: torch.Tensor, w_per_head: bool, gate: torch.Tensor, gate_col: int,
                   out: torch.Tensor, heads: int, value_dim: int, eps: float, gate_silu: bool = False):
    """Per (row, head): the scan's output (divided by its denominator where it carries one), RMS
    norm over value_dim, times ``w`` (float32 [value_dim] or [heads * value_dim]; None: no weight) and
    sigmoid(gate[:, gate_col + ...]) (``gate_silu``: times silu of it); ``out`` [rows, heads * value_dim] in the compute type."""
    _dev(raw, w, gate, out)
    rows = out.shape[0]
    ldh = value_dim + 2 if with_den else value_dim
    assert raw.dtype == torch.float32 and raw.is_contiguous() and raw.numel() == rows * heads * ldh
    assert w is None or (w.dtype == torch.float32 and w.numel() == (heads * value_dim if w_per_head else value_dim))
    assert gate.dtype == torch.float32 and gate.stride(1) == 1 and out.is_contiguous() and out.shape[1] == heads * value_dim
    _check(_fn("recurrence", "cml_head_norm_gate")(_p(raw), ldh, 1 if with_den else 0, _p(w), value_dim if w_per_head else 0,
                                                   _p(gate), gate.stride(0), gate_col, _p(out), dtype_code(out.dtype), rows,
                                                   heads, value_dim, float(eps), 1 if gate_silu else 0, _stream()), "head_norm_gate")


def rotate_rows_(x: torch.Tensor, col0: int, heads: int, head_dim: int, rotary_dim: int, interleaved: bool, inv_freq, amp: float,
                 row_pos, scaled_from: int | None = None, scale: float = 1.0):
    """In place on float32 rows: the ``heads`` heads of ``head_dim`` channels from column ``col0`` have their first
    ``rotary_dim`` channels turned by position * inv_freq (pairs of neighbours if ``interleaved``, else of the two halves;
    sines and cosines times ``amp``); heads from number ``scaled_from`` on are then multiplied by ``scale``."""
    _dev(x, inv_freq, row_pos)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and col0 + heads * head_dim <= x.shape[1]
    assert rotary_dim == 0 or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2)
    _check(_fn("recurrence", "cml_rotate_rows")(_p(x), x.stride(0), col0, x.shape[0], heads, head_dim, int(rotary_dim),
                                                1 if interleaved else 0, _p(inv_freq), float(amp), _p(row_pos),
                                                heads if scaled_from is None else int(scaled_from), float(scale), _stream()),
           "rotate_rows")


def retention_scan(proj: torch.Tensor, cols: tuple, decay: torch.Tensor, state: torch.Tensor, seq_row0, seq_new, seq_start,
                   seq_slot, out: torch.Tensor, n_seqs: int, heads: int, key_dim: int, value_dim: int):
    """Retention over each sequence's new rows: S <- decay[head] S + k v^T, out = S^T q. ``cols``: columns of q, k, v in
    ``proj`` (float32; q and k turned and scaled already); ``state`` float32 [slots, heads, value_dim, key_dim] (column by
    column) is read and replaced; ``out`` float32 [rows, heads * value_dim]."""
    _dev(proj, decay, state, seq_row0, seq_new, seq_start, seq_slot, out)
    for t in (proj, decay, state, out):
        assert t.dtype == torch.float32 and t.stride(-1) == 1
    assert decay.numel() == heads and state.is_contiguous() and state.shape[1:] == (heads, value_dim, key_dim)
    assert out.is_contiguous() and out.shape[1] == heads * value_dim
    q_col, k_col, v_col = cols
    _check(_fn("recurrence", "cml_retention_scan")(_p(proj), proj.stride(0), q_col, k_col, v_col, _p(decay), _p(state), _p(seq_row0),
                                                   _p(seq_new), _p(seq_start), _p(seq_slot), _p(out), n_seqs, heads, key_dim,
                                                   value_dim, _stream()), "retention_scan")


# ---------------------------------------------------------------------------------------
# windowed attention with keys and values of different sizes

def qk_norm_kv_write(proj: torch.Tensor, q_w, k_w, eps: float, row_seq, row_pos, table, q_out, k_pages, v_pages,
                     heads: int, kv_heads: int, key_dim: int, value_dim: int, maps: int = 1):
    """From ``proj`` (float32 rows: q, k, v): q and k RMS-normed per head with the weights ``q_w``,
    ``k_w`` (None: as they are); q to ``q_out``, k and v into their pages, all in the compute type. ``maps`` > 1: every q
    and k head is ``maps`` score maps of ``key_dim`` channels side by side, each normed on its own (the cache's key rows
    have ``maps * key_dim`` channels)."""
    _dev(proj, q_w, k_w, row_seq, row_pos, table, q_out, k_pages, v_pages)
    rows = q_out.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1
    assert proj.shape[1] >= maps * heads * key_dim + kv_heads * (maps * key_dim + value_dim)
    assert q_out.is_contiguous() and q_out.shape[1] == maps * heads * key_dim and k_pages.dtype == q_out.dtype == v_pages.dtype
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    assert k_pages.shape[1:] == (kv_heads, PAGE, maps * key_dim) and v_pages.shape[1:] == (kv_heads, PAGE, value_dim)
    norm = q_w is not None
    if norm:
        assert q_w.numel() == key_dim and k_w.numel() == key_dim and q_w.dtype == k_w.dtype
    _check(_fn("attention_window", "cml_qk_norm_kv_write")(
        _p(proj), proj.stride(0), _p(q_w), _p(k_w), dtype_code(q_w.dtype) if norm else dtype_code(q_out.dtype), 1 if norm else 0,
        float(eps), _p(row_seq), _p(row_pos), _p(table), table.shape[1], _p(q_out), _p(k_pages), _p(v_pages),
        dtype_code(q_out.dtype), rows, heads, kv_heads, key_dim, value_dim, int(maps), _stream()), "qk_norm_kv_write")


def window_attention(q, k_pages, v_pages, table, row_seq, row_pos, r1, r2, gate, gate_col: int, out, heads: int,
                     kv_heads: int, key_dim: int, value_dim: int, window: int, scale: float, chunk: int = 0, sink=None,
                     gate_per_head: bool = False, softcap: float = 0.0, difference=None, keep_first: int = 0,
                     values_in_keys: bool = False):
    """``softcap`` c > 0: the scaled score becomes c tanh(score / c). ``difference`` = (lambda, eps, out_scale): every head
    has two score maps (q and the key rows hold both, ``key_dim`` channels each), out = rmsnorm_eps(a1 - lambda a2) * out_scale
    per head (differential attention).
    out[r, head] = softmax_j((q . k_j) scale - r1 ln(1 + r2 (i - j))) V over the last ``window`` keys
    (0: all) and, with ``chunk``, only those of the row's own block of ``chunk`` positions; ``sink`` (float32
    [heads]): one more term exp(sink) in the denominator; times sigmoid(gate[r, gate_col + ...]) where ``gate``
    (float32) is given: a number per channel of every head, or per head. ``keep_first`` n (with a window): the first n
    keys of the sequence stay visible whatever the window. ``values_in_keys``: a value is the first ``value_dim`` channels
    of its key row (``v_pages`` is ``k_pages``)."""
    _dev(q, k_pages, v_pages, table, row_seq, row_pos, r1, r2, gate, out, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == heads and sink.is_contiguous())
    rows = q.shape[0]
    assert q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype == k_pages.dtype == v_pages.dtype
    maps = 2 if difference is not None else 1
    lam, d_eps, d_scale = difference if difference is not None else (0.0, 0.0, 1.0)
    assert out.shape == (rows, heads * value_dim) and q.shape[1] == maps * heads * key_dim
    assert k_pages.shape[1:] == (kv_heads, PAGE, maps * key_dim)
    if values_in_keys:
        assert v_pages.data_ptr() == k_pages.data_ptr() and value_dim <= maps * key_dim
    else:
        assert v_pages.shape[1:] == (kv_heads, PAGE, value_dim)
    if r1 is not None:
        assert r1.dtype == torch.float32 and r2.dtype == torch.float32 and r1.numel() == heads and r2.numel() == heads
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1
    _check(_fn("attention_window", "cml_window_attention")(
        _p(q), _p(k_pages), _p(v_pages), dtype_code(q.dtype), _p(table), table.shape[1], _p(row_seq), _p(row_pos), _p(r1),
        _p(r2), _p(gate), gate.stride(0) if gate is not None else 0, gate_col, _p(out), rows, heads, kv_heads, key_dim,
        value_dim, int(window or 0), float(scale), int(chunk or 0), _p(sink), 1 if gate_per_head else 0, maps, float(softcap or 0.0),
        float(lam), float(d_eps), float(d_scale), int(keep_first or 0), maps * key_dim if values_in_keys else value_dim,
        _stream()), "window_attention")


def qkv_prepare(proj: torch.Tensor, q_w, k_w, norm_mode: int, eps: float, inv_freq, rotary_dim: int, interleaved: bool,
                row_seq, row_pos, table, q_out, k_pages, v_pages, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                extra_out=None, bias=None, amplitude: float = 1.0):
    """``bias`` (float32, one number per column of q, k, v and the extra columns): added to the summed row before the norms;
    ``amplitude`` multiplies every sine and cosine.
    From ``proj`` (float32 rows: q, k, v; [rows, n] or split sums [splits, rows, n], added here): RMS norm of q and k (``norm_mode`` 0 none, 1 per head with weights
    [key_dim], 2 over the whole projection with weights [heads * key_dim] and [kv_heads * key_dim]), then the
    first ``rotary_dim`` channels of every head rotated by position * inv_freq (pairs of neighbours if
    ``interleaved``, else of the two halves); q to ``q_out``, k and v into their pages, in the compute type.
    ``extra_out`` (float32 [rows, e]): the e columns behind v (an output gate's logits), summed over the splits."""
    _dev(proj, q_w, k_w, inv_freq, row_seq, row_pos, table, q_out, k_pages, v_pages, extra_out)
    rows = q_out.shape[0]
    if proj.dim() == 2:
        proj = proj.unsqueeze(0)
    assert proj.dtype == torch.float32 and proj.stride(2) == 1 and proj.shape[1] == rows
    extra = extra_out.shape[1] if extra_out is not None else 0
    assert extra_out is None or (extra_out.dtype == torch.float32 and extra_out.is_contiguous() and extra_out.shape[0] == rows)
    assert proj.shape[2] >= heads * key_dim + kv_heads * (key_dim + value_dim) + extra
    assert q_out.is_contiguous() and q_out.shape[1] == heads * key_dim and k_pages.dtype == q_out.dtype == v_pages.dtype
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    assert k_pages.shape[1:] == (kv_heads, PAGE, key_dim) and v_pages.shape[1:] == (kv_heads, PAGE, value_dim)
    if norm_mode:
        per = key_dim if norm_mode == 1 else heads * key_dim
        assert q_w.numel() == per and k_w.numel() == (key_dim if norm_mode == 1 else kv_heads * key_dim) and q_w.dtype == k_w.dtype
    if rotary_dim:
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2
    if bias is not None:
        _dev(bias)
        assert bias.dtype == torch.float32 and bias.is_contiguous()
        assert bias.numel() == heads * key_dim + kv_heads * (key_dim + value_dim) + extra
    _check(_fn("attention_window", "cml_qkv_prepare")(
        _p(proj), proj.stride(1), proj.shape[0], proj.stride(0), extra, _p(extra_out), _p(q_w), _p(k_w), dtype_code(q_w.dtype) if norm_mode else dtype_code(q_out.dtype), int(norm_mode),
        float(eps), _p(inv_freq), int(rotary_dim), 1 if interleaved else 0, _p(row_seq), _p(row_pos), _p(table), table.shape[1],
        _p(q_out), _p(k_pages), _p(v_pages), dtype_code(q_out.dtype), rows, heads, kv_heads, key_dim, value_dim, _p(bias),
        float(amplitude), _stream()), "qkv_prepare")


def latent_prepare(proj: torch.Tensor, c_w: torch.Tensor, eps: float, inv_freq, interleaved: bool, amplitude: float, row_seq,
                   row_pos, table, q_plain, q_full, k_pages, heads: int, plain_dim: int, rot_dim: int, rank: int, extra_out=None):
    """The rows of a step for attention over a latent. ``proj`` (float32 [rows, n] or split sums [splits, rows, n], added
    here) holds q (``heads`` x [``plain_dim`` unturned, ``rot_dim`` turned]), then ``rank`` + ``rot_dim`` columns of the down
    projection, then the columns of ``extra_out`` (float32 [rows, e]). Writes the unturned query parts to ``q_plain``
    [rows, heads * plain_dim], the turned ones to channels ``rank``.. of every head of ``q_full`` [rows, heads * (rank +
    rot_dim)], and [rmsnorm(down[:rank]) * c_w, turned(down[rank:])] into the sequence's page row, all in the compute type."""
    _dev(proj, c_w, inv_freq, row_seq, row_pos, table, q_plain, q_full, k_pages, extra_out)
    rows = q_full.shape[0]
    if proj.dim() == 2:
        proj = proj.unsqueeze(0)
    extra = extra_out.shape[1] if extra_out is not None else 0
    assert proj.dtype == torch.float32 and proj.stride(2) == 1 and proj.shape[1] == rows
    assert proj.shape[2] >= heads * (plain_dim + rot_dim) + rank + rot_dim + extra
    assert extra_out is None or (extra_out.dtype == torch.float32 and extra_out.is_contiguous() and extra_out.shape[0] == rows)
    assert q_plain.is_contiguous() and q_plain.shape == (rows, heads * plain_dim) and q_full.is_contiguous()
    assert q_full.shape == (rows, heads * (rank + rot_dim)) and q_plain.dtype == q_full.dtype == k_pages.dtype
    assert k_pages.is_contiguous() and k_pages.shape[1:] == (1, PAGE, rank + rot_dim) and c_w.numel() == rank
    assert rot_dim == 0 or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rot_dim // 2)
    _check(_fn("attention_latent", "cml_latent_prepare")(
        _p(proj), proj.stride(1), proj.shape[0], proj.stride(0), extra, _p(extra_out), _p(c_w), dtype_code(c_w.dtype), float(eps),
        _p(inv_freq), 1 if interleaved else 0, float(amplitude), _p(row_seq), _p(row_pos), _p(table), table.shape[1], _p(q_plain),
        _p(q_full), _p(k_pages), dtype_code(q_full.dtype), rows, heads, plain_dim, rot_dim, rank, _stream()), "latent_prepare")


LATENT_PROMPT_ROWS = 64        # (token, head) query rows of a block of the prompt kernel; LA_ROWS in attention_latent.cu


def latent_prompt_tokens(heads: int) -> int:
    """Tokens of a query tile of ``latent_prompt``."""
    return 1 if heads >= LATENT_PROMPT_ROWS else LATENT_PROMPT_ROWS // heads


def latent_prompt_usable(q: torch.Tensor, rank: int, rot_dim: int) -> bool:
    """Whether ``latent_prompt`` takes these rows: bfloat16, a latent of a multiple of 32 channels up to 512 and a
    turned part of a multiple of 16, together at most 576 channels (a block's three tiles of 64 rows fill shared memory)."""
    return (q.dtype == torch.bfloat16 and 32 <= rank <= 512 and rank % 32 == 0 and rot_dim % 16 == 0
            and rank + rot_dim <= 576)


def latent_prompt(q_full, k_pages, out, table, tile_seq, tile_q0, n_tiles: int, seq_row0, seq_start, seq_new, heads: int,
                  rank: int, rot_dim: int, scale: float, sink=None, head_gate=None, gate_col: int = 0, partial=None,
                  tiles_per_split: int = 0):
    """bfloat16 prompt attention over a latent on the tensor cores (mma.sync): ``q_full`` [rows, heads * (rank + rot_dim)]
    against the sequences' cached rows [c, t] (``k_pages`` [pages, 1, 64, rank + rot_dim]), every earlier key visible;
    ``out`` [rows, heads * rank] gets the weighted latents per head, with exp(``sink``[head]) as one more term of the
    denominator and times sigmoid(``head_gate``[r, gate_col + head]). Tiles of ``latent_prompt_tokens(heads)`` tokens.
    ``partial`` (float32 [splits, rows, heads, rank + 2]; steps of one token per sequence only): a sequence's pages are
    dealt to ``splits`` blocks, ``tiles_per_split`` pages each, and a second launch merges their shares in split order."""
    _dev(q_full, k_pages, out, table, tile_seq, tile_q0, seq_row0, seq_start, seq_new, sink, head_gate)
    rows, D = q_full.shape[0], rank + rot_dim
    assert latent_prompt_usable(q_full, rank, rot_dim) and q_full.is_contiguous() and q_full.shape[1] == heads * D
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == (rows, heads * rank)
    assert k_pages.dtype == torch.bfloat16 and k_pages.is_contiguous() and k_pages.shape[1:] == (1, PAGE, D)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == heads and sink.is_contiguous())
    assert head_gate is None or (head_gate.dtype == torch.float32 and head_gate.stride(1) == 1 and head_gate.shape[0] == rows
                                 and gate_col + heads <= head_gate.shape[1])
    if partial is not None:
        _dev(partial)
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1:] == (rows, heads, rank + 2)
        assert tiles_per_split >= 1 and n_tiles == rows
    _check(_fn("attention_latent", "cml_latent_prompt")(
        _p(q_full), _p(k_pages), _p(out), _p(table), table.shape[1], _p(tile_seq), _p(tile_q0), int(n_tiles),
        1 if partial is not None else latent_prompt_tokens(heads), _p(seq_row0), _p(seq_start), _p(seq_new), _p(sink), _p(head_gate),
        head_gate.stride(0) if head_gate is not None else 0, int(gate_col), heads, rank, rot_dim, float(scale), _p(partial),
        partial.shape[0] if partial is not None else 1, int(tiles_per_split), rows, _stream()),
        "latent_prompt", 2 if partial is not None else 1)


def head_product(x: torch.Tensor, x_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int):
    """out[r, h * out_head_stride + n] = sum_k x[r, h * x_head_stride + k] * w[h, n, k] for every head h: one product per
    head, float32 accumulation. ``w`` [heads, N, K] contiguous; ``x`` and ``out`` 2-d in the compute type, rows any stride."""
    _dev(x, w, out)
    heads, n, k = w.shape
    rows = x.shape[0]
    assert w.is_contiguous() and x.dtype == w.dtype == out.dtype and x.stride(1) == 1 and out.stride(1) == 1
    assert out.shape[0] == rows and (heads - 1) * x_head_stride + k <= x.shape[1] and (heads - 1) * out_head_stride + n <= out.shape[1]
    _check(_fn("attention_latent", "cml_head_product")(_p(x), x.stride(0), int(x_head_stride), _p(w), _p(out), out.stride(0),
                                                      int(out_head_stride), dtype_code(x.dtype), rows, heads, n, k, _stream()),
           "head_product")


# ---------------------------------------------------------------------------------------
# routed feed-forwards

def route_topk(logits: torch.Tensor, top: int, softmax: bool, renorm: bool, ids: torch.Tensor, wts: torch.Tensor,
               correction=None, groups: int = 1, keep_groups: int = 1, weight_scale: float = 1.0):
    """The ``top`` largest logits of every row: their expert ids and weights (sigmoid of the logit, or its softmax
    over all experts; ``renorm``: divided by the chosen weights' sum; times ``weight_scale``). logits float32 [rows,
    experts], or split sums [splits, rows, experts] that are added first. ``correction`` (float32 [experts]) is added
    to the scores for the choice only; with ``groups`` > 1 the experts form that many equal groups of neighbours and
    only the ``keep_groups`` groups with the largest choice score of a member can be chosen from."""
    _dev(logits, ids, wts, correction)
    assert correction is None or (correction.dtype == torch.float32 and correction.is_contiguous())
    if logits.dim() == 2:
        logits = logits.unsqueeze(0)
    _, rows, experts = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(2) == 1 and ids.dtype == torch.int32 and wts.dtype == torch.float32
    assert ids.numel() == rows * top == wts.numel() and ids.is_contiguous() and wts.is_contiguous()
    _check(_fn("experts", "cml_route_topk")(_p(logits), logits.stride(1), logits.shape[0], logits.stride(0), rows, experts, int(top), 1 if softmax else 0,
                                            1 if renorm else 0, _p(correction), int(groups), int(keep_groups), float(weight_scale),
                                            _p(ids), _p(wts), _stream()), "route_topk")


EXPERT_TILE_ROWS, EXPERT_TILE_ROWS_TC = 64, 128      # rows of a tile of the grouped products: CUDA cores, tensor cores


def expert_plan(ids: torch.Tensor, experts: int, rank, counts, offsets, tile_first, tile_rows: int = EXPERT_TILE_ROWS):
    """Orders the (row, choice) pairs by expert: ``rank`` of each pair among its expert's, ``counts`` per expert,
    ``offsets`` [experts + 1] and the first tile (of ``tile_rows`` rows) of every expert's stretch ``tile_first``
    [experts + 1]."""
    _dev(ids, rank, counts, offsets, tile_first)
    assert all(t.dtype == torch.int32 and t.is_contiguous() for t in (ids, rank, counts, offsets, tile_first))
    assert rank.numel() == ids.numel() and counts.numel() >= experts and offsets.numel() > experts and tile_first.numel() > experts
    _check(_fn("experts", "cml_expert_plan")(_p(ids), ids.numel(), experts, _p(rank), _p(counts), _p(offsets), _p(tile_first),
                                             int(tile_rows), _stream()), "expert_plan", launches=2)


def expert_gather(x: torch.Tensor, ids, wts, rank, offsets, top: int, scale_input: bool, xs: torch.Tensor, pos_of_pair,
                  real_experts: int = 1 << 30):
    """xs[offsets[expert] + rank] = x[row] (times the pair's weight if ``scale_input``); ``pos_of_pair`` keeps the place.
    Pairs of experts ``real_experts`` and up (identity experts) are not copied."""
    _dev(x, ids, wts, rank, offsets, xs, pos_of_pair)
    pairs = ids.numel()
    assert x.stride(1) == 1 and xs.is_contiguous() and xs.shape == (pairs, x.shape[1]) and xs.dtype == x.dtype
    _check(_fn("experts", "cml_expert_gather")(_p(x), dtype_code(x.dtype), x.stride(0), x.shape[1], _p(ids), _p(wts), _p(rank),
                                               _p(offsets), pairs, int(top), 1 if scale_input else 0, int(real_experts), _p(xs), _p(pos_of_pair),
                                               _stream()), "expert_gather")


def expert_gemm(a: torch.Tensor, w: torch.Tensor, w2, out: torch.Tensor, offsets, tile_first, act=None):
    """Per expert e: out[stretch e] = a[stretch e] @ w[e].T (float32), or with ``w2`` the gated activation ``act``
    (``GateAct``; None: SiLU gating) of (a @ w[e].T, a @ w2[e].T) in the compute type. w [experts, n, k]; the stretches
    are ``offsets``."""
    _dev(a, w, w2, out, offsets, tile_first)
    pairs, k = a.shape
    experts, n, k2 = w.shape
    assert k == k2 and a.is_contiguous() and w.is_contiguous() and a.dtype == w.dtype and out.is_contiguous()
    assert out.shape == (pairs, n) and out.dtype == (a.dtype if w2 is not None else torch.float32)
    assert w2 is None or (w2.shape == w.shape and w2.is_contiguous() and w2.dtype == w.dtype)
    if w2 is not None:
        _gate_act("experts", act)
    _check(_fn("experts", "cml_expert_gemm")(_p(a), _p(w), _p(w2), dtype_code(a.dtype), _p(out), pairs, n, k, experts,
                                             _p(offsets), _p(tile_first), _stream()), "expert_gemm")


def gemm_tc_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, offsets, tile_first, err: torch.Tensor,
                    act=None):
    """The grouped product on the tensor cores (bfloat16): per expert e, out[stretch e] = a[stretch e] @ w[e].T with
    epilogue TC_STORE_F32 (float32 out), TC_STORE (bfloat16) or TC_SWIGLU (w[e] packed gate/up rows in groups of 16,
    out [rows, n / 2] bfloat16). ``offsets``, ``tile_first``: from ``expert_plan`` with tiles of 128 rows."""
    _dev(a, w, out, offsets, tile_first, err)
    rows, k = a.shape
    experts, n, k2 = w.shape
    assert k == k2 and a.dtype == w.dtype == torch.bfloat16 and w.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1
    assert epilogue in (TC_STORE, TC_STORE_F32, TC_SWIGLU)
    assert out.shape == (rows, n // 2 if epilogue == TC_SWIGLU else n)
    assert out.dtype == (torch.float32 if epilogue == TC_STORE_F32 else torch.bfloat16)
    bn = 256 if n % 256 == 0 and n >= 1024 else 128
    if epilogue == TC_SWIGLU:
        _gate_act("gemm_tc", act)
    _check(_fn("gemm_tc", "cml_gemm_tc_grouped")(_p(a), a.stride(0), rows, _p(w), k, experts, n, k, _p(out), out.stride(0),
                                                 epilogue, bn, _p(offsets), _p(tile_first), _p(err), _stream()), "gemm_tc_grouped")


def expert_combine(y: torch.Tensor, pos_of_pair, wts, top: int, scale_output: bool, shared, out: torch.Tensor,
                   identity=None):
    """out[row] = shared[row] + sum over the row's choices of y[place of the pair] (times its weight if
    ``scale_output``); ``shared`` float32 [rows, hidden] or [splits, rows, hidden] or None. ``identity`` = (ids,
    real_experts, rows): a choice of an expert ``real_experts`` or up adds ``rows[row]`` (float32 or bfloat16
    [rows, hidden]) times its weight instead."""
    _dev(y, pos_of_pair, wts, shared, out)
    i_ids, i_real, i_rows = identity if identity is not None else (None, 0, None)
    if identity is not None:
        _dev(i_ids, i_rows)
        assert i_rows.shape == out.shape and i_rows.is_contiguous() and i_ids.dtype == torch.int32
    rows, hidden = out.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (rows * top, hidden) and out.is_contiguous()
    splits, stride = 0, 0
    if shared is not None:
        if shared.dim() == 2:
            shared = shared.unsqueeze(0)
        assert shared.dtype == torch.float32 and shared.shape[1:] == (rows, hidden) and shared.stride(2) == 1 and shared.stride(1) == hidden
        splits, stride = shared.shape[0], shared.stride(0)
    _check(_fn("experts", "cml_expert_combine")(_p(y), _p(pos_of_pair), _p(wts), int(top), 1 if scale_output else 0, _p(shared),
                                                splits, stride, _p(i_ids), int(i_real), _p(i_rows),
                                                dtype_code(i_rows.dtype) if i_rows is not None else 0, _p(out), rows, hidden,
                                                _stream()), "expert_combine")


TC_STORE, TC_STORE_F32, TC_ADD_F32, TC_SWIGLU, TC_T_PARTIAL, TC_T_SWIGLU = 0, 1, 2, 3, 4, 5


def _tc_operand(t: torch.Tensor) -> bool:
    """Whether TMA can fetch tiles of ``t`` ([rows, K] bfloat16, K-major): 16-byte aligned base and
    row stride, so K and the stride are multiples of 8. Remembered on the tensor: weights and
    the workspace's views are the same objects step after step."""
    try:
        return t._cml_tc_operand
    except AttributeError:
        ok = (t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] % 8 == 0 and t.stride(1) == 1
              and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0)
        t._cml_tc_operand = ok
        return ok


def gemm_tc_usable(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands ([rows, K] bfloat16, K-major): TMA
    needs 16-byte aligned bases and row strides, so K and the strides must be multiples of 8."""
    return _tc_operand(a) and _tc_operand(b) and a.shape[1] == b.shape[1]


def gemm_tc(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, epilogue: int, bn: int, splits: int, err: torch.Tensor, act=None):
    """D = a @ b.T on the tensor cores (see gemm_tc.cu). Epilogues 0..3 write c[row of a][row of b];
    4 and 5 are transposed: c[split][row of b][row of a] partial sums, or SwiGLU of packed a rows. ``act``
    (``GateAct``; None: SiLU gating): the activation of the gated epilogues."""
    _dev(a, b, c, err)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc: operands must be bfloat16 [rows, K] with K and the row strides multiples of 8 "
                          "and 16-byte aligned bases")
    assert c.stride(-1) == 1
    ldc = c.stride(-2)
    if epilogue in (TC_SWIGLU, TC_T_SWIGLU):
        _gate_act("gemm_tc", act)
    _check(_fn("gemm_tc", "cml_gemm_tc")(_p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], a.shape[1],
                                        _p(c), ldc, epilogue, bn, splits, _p(err), _stream()), "gemm_tc")


class RowScale:
    """What a norm left undone when the product before it wrote the norm's output: the rows of
    that output lack the factor rsqrt(sum over parts of sumsq[part][row] / hidden + eps).
    The product that reads those rows applies it to its own output rows (a product is linear
    in its input rows), or ``scale_rows`` applies it in place."""

    def __init__(self, sumsq: torch.Tensor, hidden: int, eps: float):
        assert sumsq.dim() == 2 and sumsq.dtype == torch.float32 and sumsq.is_contiguous()
        self.sumsq, self.hidden, self.eps = sumsq, int(hidden), float(eps)


def gemm_tc_pair(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, epilogue: int, err: torch.Tensor,
                 row_scale: "RowScale | None" = None, act=None):
    """c[row of a][row of b] (op)= a @ b.T with epilogues 0..3 of ``gemm_tc``, on tiles of
    256 x 256 that the two blocks of a cluster share (tcgen05 cta_group::2): the kernel for
    products with many rows of ``a``. ``row_scale``: the scale the rows of ``a`` still lack."""
    _dev(a, b, c, err)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc_pair: operands must be bfloat16 [rows, K] with K and the row strides multiples "
                          "of 8 and 16-byte aligned bases")
    assert c.stride(-1) == 1 and epilogue in (TC_STORE, TC_STORE_F32, TC_ADD_F32, TC_SWIGLU)
    sumsq, parts, hidden, eps = None, 0, 0, 0.0
    if row_scale is not None:
        sumsq, hidden, eps = row_scale.sumsq, row_scale.hidden, row_scale.eps
        _dev(sumsq)
        parts = sumsq.shape[0]
        assert sumsq.shape[1] == a.shape[0]
    if epilogue == TC_SWIGLU:
        _gate_act("gemm_tc", act)
    _check(_fn("gemm_tc", "cml_gemm_tc_pair")(_p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], a.shape[1],
                                             _p(c), c.stride(-2), epilogue, _p(err), _p(sumsq), parts, hidden, eps,
                                             _stream()), "gemm_tc_pair")


def pair_partial_splits(k: int, wanted: int) -> int:
    """How many splits of K ``gemm_tc_pair_partial`` makes when asked for ``wanted``: k-blocks of
    64 are dealt out evenly and no split stays empty."""
    blocks = (k + 63) // 64
    per = (blocks + max(1, min(wanted, blocks)) - 1) // max(1, min(wanted, blocks))
    return (blocks + per - 1) // per


def gemm_tc_pair_partial(a: torch.Tensor, b: torch.Tensor, part: torch.Tensor, err: torch.Tensor,
                         row_scale: "RowScale | None" = None):
    """part[s] (float32 [splits, rows of a, rows of b]) = the share of a @ b.T of the s-th split of
    K, on the two-block tiles of ``gemm_tc_pair``; the splits are work items of their own, which
    gives a product of a few hundred rows enough of them for every SM. ``part.shape[0]`` must be
    a count that ``pair_partial_splits`` returns."""
    _dev(a, b, part, err)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc_pair_partial: operands must be bfloat16 [rows, K] with K and the row strides "
                          "multiples of 8 and 16-byte aligned bases")
    assert part.dtype == torch.float32 and part.dim() == 3 and part.stride(2) == 1
    assert part.shape[1:] == (a.shape[0], b.shape[0])
    sumsq, parts, hidden, eps = None, 0, 0, 0.0
    if row_scale is not None:
        sumsq, hidden, eps = row_scale.sumsq, row_scale.hidden, row_scale.eps
        _dev(sumsq)
        parts = sumsq.shape[0]
        assert sumsq.shape[1] == a.shape[0]
    _check(_fn("gemm_tc", "cml_gemm_tc_pair_partial")(
        _p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], a.shape[1], _p(part), part.stride(1),
        part.stride(0), part.shape[0], _p(err), _p(sumsq), parts, hidden, eps, _stream()), "gemm_tc_pair_partial")


def gemm_tc_pair_add_norm(a: torch.Tensor, b: torch.Tensor, h: torch.Tensor, err: torch.Tensor, norm_w: torch.Tensor,
                          eps: float, x_out: torch.Tensor, sumsq: torch.Tensor) -> RowScale:
    """h (float32 [rows, out]) += a @ b.T, and the first half of the RMS norm that reads h next:
    x_out = bfloat16(h * norm_w) and the sums of squares of every row, one per tile of 256
    columns, in ``sumsq`` (float32 [ceil(out / 256), rows]). Returns the scale the rows of
    x_out still lack."""
    _dev(a, b, h, err, norm_w, x_out, sumsq)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc_pair_add_norm: operands must be bfloat16 [rows, K] with K and the row strides "
                          "multiples of 8 and 16-byte aligned bases")
    rows, n = a.shape[0], b.shape[0]
    assert h.dtype == torch.float32 and h.shape == (rows, n) and h.stride(1) == 1
    assert x_out.dtype == torch.bfloat16 and x_out.shape == (rows, n) and x_out.stride(1) == 1
    assert norm_w.numel() == n and norm_w.is_contiguous()
    assert sumsq.dtype == torch.float32 and sumsq.is_contiguous() and sumsq.shape == ((n + 255) // 256, rows)
    _check(_fn("gemm_tc", "cml_gemm_tc_pair_add_norm")(
        _p(a), a.stride(0), rows, _p(b), b.stride(0), n, a.shape[1], _p(h), h.stride(0), _p(err), _p(norm_w),
        dtype_code(norm_w.dtype), _p(x_out), x_out.stride(0), _p(sumsq), _stream()), "gemm_tc_pair_add_norm")
    return RowScale(sumsq, n, eps)


def scale_rows(x: torch.Tensor, row_scale: RowScale):
    """x[r] *= the scale its rows still lack, in place."""
    _dev(x, row_scale.sumsq)
    assert x.dim() == 2 and x.stride(1) == 1 and row_scale.sumsq.shape[1] == x.shape[0]
    _check(_fn("rowwise", "cml_scale_rows")(_p(x), dtype_code(x.dtype), x.stride(0), x.shape[0], x.shape[1],
                                           _p(row_scale.sumsq), row_scale.sumsq.shape[0], row_scale.hidden,
                                           row_scale.eps, _stream()), "scale_rows")


def attn_heads_per_warp(heads_per_cta: int, decode: bool) -> int:
    """Heads of one token that a warp of the float attention kernel owns: in prefill as many of
    4, 2, 1 as divide the block's heads (a key read from shared memory serves them all). 0 names
    the decode kernel, whose four warps share every page by keys and all work on the block's 2 or
    4 heads; a decode step on single heads gives each its own warp."""
    if decode:
        return 0 if heads_per_cta in (2, 4) else 1
    return 4 if heads_per_cta % 4 == 0 else 2 if heads_per_cta % 2 == 0 else 1


def attn_tiling(n_heads: int, n_kv_heads: int, decode: bool) -> tuple[int, int, int]:
    """(rows_per_tile, heads_per_cta, head_chunks) of the float attention kernel. Prefill: at most
    16 warps, each with one token and ``attn_heads_per_warp`` of its heads; the heads of a kv group
    are cut in chunks if above 16. Decode: one token and 2 or 4 heads of a kv group per block."""
    group = n_heads // n_kv_heads
    if decode:
        hpc = 1 if group == 1 else 2 if group == 2 else 4
        return 1, hpc, (group + hpc - 1) // hpc
    chunks = (group + 15) // 16
    hpc = (group + chunks - 1) // chunks
    rows = max(1, 16 * attn_heads_per_warp(hpc, False) // hpc)
    return rows, hpc, chunks


def attn_simt_smem_bytes(head_dim: int, rows_per_tile: int, heads_per_cta: int, decode: bool) -> int:
    """Shared memory of a block of the float attention kernel with this tiling."""
    f = _fn("attention_simt", "cml_attn_simt_smem_bytes")
    f.restype = c_long
    return int(f(head_dim, rows_per_tile, heads_per_cta, attn_heads_per_warp(heads_per_cta, decode)))


def attn_partial_floats(n_rows: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return n_rows * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def attn_paged_simt(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, n_tiles, seq_row0, seq_start, seq_new,
                    n_rows, n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, head_chunks, n_splits,
                    window, scale, partial, heads_per_warp=None):
    """Attention of packed query rows over the paged cache (float arithmetic). ``q`` may be a
    column slice of a wider matrix (its row stride is used). ``heads_per_warp``: by default what
    ``attn_tiling`` assumed (one where a tile is a single row)."""
    if heads_per_warp is None:
        heads_per_warp = attn_heads_per_warp(heads_per_cta, rows_per_tile == 1)
    _dev(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, seq_row0, seq_start, seq_new, partial)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == v_pages.dtype
    assert k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
    if n_splits > 1:
        assert partial is not None and partial.dtype == torch.float32
        assert partial.numel() >= attn_partial_floats(n_rows, n_heads, head_dim, n_splits)
    _check(_fn("attention_simt", "cml_attn_paged_simt")(
        _p(q), q.stride(0), _p(out), out.stride(0), dtype_code(q.dtype), _p(k_pages), _p(v_pages), _p(block_table),
        block_table.shape[1], _p(tile_seq), _p(tile_q0), n_tiles, _p(seq_row0), _p(seq_start), _p(seq_new), n_rows,
        n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, heads_per_warp, head_chunks, n_splits,
        int(window or 0), float(scale), _p(partial), _stream()), "attn_paged_simt", 2 if n_splits > 1 else 1)


def attn_mma_tiling(n_heads: int, n_kv_heads: int, decode: bool) -> tuple[int, int, int]:
    """(rows_per_tile, heads_per_cta, head_chunks) of the mma.sync attention kernel: the 16
    rows of an MMA hold the grouped heads of one kv head times a few consecutive tokens."""
    group = n_heads // n_kv_heads
    chunks = (group + 15) // 16
    hpc = (group + chunks - 1) // chunks
    rows = 1 if decode else max(1, 16 // hpc)
    return rows, hpc, chunks


def attn_mma_usable(q: torch.Tensor, head_dim: int) -> bool:
    return q.dtype == torch.bfloat16 and head_dim in (64, 128) and q.stride(0) % 2 == 0


def attn_paged_mma(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, n_tiles, seq_row0, seq_start, seq_new,
                   n_rows, n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, head_chunks, n_splits,
                   window, scale, partial):
    """bfloat16 attention of packed query rows over the paged cache on the tensor cores."""
    _dev(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, seq_row0, seq_start, seq_new, partial)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == torch.bfloat16
    assert k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
    tickets = None
    if n_splits > 1:
        assert partial is not None and partial.dtype == torch.float32
        assert partial.numel() >= attn_partial_floats(n_rows, n_heads, head_dim, n_splits)
        tickets = zeroed_scratch(q.device, "attention_tickets", 4 * n_tiles * n_kv_heads * head_chunks)
    _check(_fn("attention_mma", "cml_attn_paged_mma")(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1],
        _p(tile_seq), _p(tile_q0), n_tiles, _p(seq_row0), _p(seq_start), _p(seq_new), n_rows, n_heads, n_kv_heads,
        head_dim, rows_per_tile, heads_per_cta, head_chunks, n_splits, int(window or 0), float(scale), _p(partial),
        _p(tickets), _stream()), "attn_paged_mma")


def attn_decode_fused_usable(partial, out, head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    return (partial is not None and partial.dtype == torch.float32 and out.dtype == torch.bfloat16
            and head_dim in (64, 128) and n_heads // n_kv_heads <= 16 and out.stride(0) % 2 == 0)


def attn_decode_fused_splits(n_splits: int, n_heads: int, n_kv_heads: int, head_dim: int) -> int:
    """The number of blocks per cluster the fused decode kernel can take, at most ``n_splits``:
    block 0 keeps the ranges of all blocks in shared memory beside its own cache tiles."""
    group = n_heads // n_kv_heads
    stages = 4 * 3 * 2 * 32 * head_dim * 2
    n_splits = max(1, min(8, n_splits))
    while n_splits > 1 and stages + n_splits * group * (head_dim + 2) * 4 + 8 * 1024 > 227 * 1024:
        n_splits -= 1
    return n_splits


def attn_decode_fused(partial, out, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq, rotary_dim: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool, window: int, scale: float,
                      n_splits: int):
    """Decode attention in one launch from the partial sums [splits, rows, width] of the q/k/v
    product: sums them, rotates q and the new key, writes the new key and value to the cache
    (``write_kv``) and attends every row (one new token of a sequence each) over its cache,
    the keys split over the ``n_splits`` (at most 8) blocks of a cluster."""
    _dev(partial, out, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq)
    assert partial.dim() == 3 and partial.is_contiguous() and out.stride(1) == 1
    assert k_pages.dtype == torch.bfloat16 and k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim)
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and 1 <= n_splits <= 8
    rows = partial.shape[1]
    _check(_fn("attention_mma", "cml_attn_decode_fused")(
        _p(partial), partial.shape[0], partial.stride(0), partial.shape[2], rows, _p(row_pos), _p(row_seq),
        _p(block_table), block_table.shape[1], _p(k_pages), _p(v_pages), _p(inv_freq), rotary_dim, n_heads, n_kv_heads,
        head_dim, 1 if write_kv else 0, int(window or 0), float(scale), n_splits, _p(out), out.stride(0), _stream()),
        "attn_decode_fused")


def attn_tc_tiling(n_heads: int, n_kv_heads: int) -> tuple[int, int, int]:
    """(rows_per_tile, heads_per_cta, head_chunks) of the tcgen05 prefill attention kernel: the
    128 lanes of tensor memory hold the grouped heads of one kv head times consecutive tokens."""
    group = n_heads // n_kv_heads
    chunks = (group + 15) // 16
    hpc = (group + chunks - 1) // chunks
    return max(1, 128 // hpc), hpc, chunks


def attn_tc_usable(q: torch.Tensor, out: torch.Tensor, head_dim: int, value_dim: int | None = None) -> bool:
    return (q.dtype == torch.bfloat16 and head_dim in (64, 128) and (value_dim or head_dim) in (64, 128) and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def attn_prefill_tc(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, n_tiles, seq_row0, seq_start, seq_new,
                    n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, head_chunks, window, scale, err,
                    r1=None, r2=None, chunk: int = 0, sink=None, head_gate=None, gate_col: int = 0, maps: int = 1,
                    softcap: float = 0.0, value_dim: int | None = None, keep_first: int = 0):
    """``keep_first`` n (with ``window``): the first n keys of a sequence stay visible to all its later queries.
    bfloat16 prefill attention of packed query rows over the paged cache with tcgen05.mma. ``r1``, ``r2``
    (float32 [heads]): the score of key j for query i loses r1 ln(1 + r2 (i - j)). ``chunk``: queries see only the
    keys of their own block of ``chunk`` positions. ``sink`` (float32 [heads]): one more term exp(sink) in the
    denominator. ``head_gate`` (float32 [rows, ...]): head h of row r times sigmoid(head_gate[r, gate_col + h]).
    ``maps`` score maps per head: q rows hold [head, map, head_dim], the key rows of the cache the maps' channels side by
    side, the values are shared, and ``out`` (float32 or bfloat16) gets [head, map, head_dim], every map's attention by
    itself (``maps_difference`` combines two; with more than one map the probabilities enter the P V product as two
    bfloat16 parts each, since the maps' outputs are subtracted afterwards). ``softcap`` c > 0: the scaled score becomes c tanh(score / c).
    ``value_dim``: channels of a value (64 or 128) where they differ from a key's ``head_dim``; the output rows then hold
    [head, map, value_dim]."""
    value_dim = int(value_dim or head_dim)
    _dev(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, seq_row0, seq_start, seq_new, err, r1, r2, sink, head_gate)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads and sink.is_contiguous())
    assert head_gate is None or (head_gate.dtype == torch.float32 and head_gate.stride(1) == 1 and head_gate.shape[0] == q.shape[0]
                                 and gate_col + n_heads <= head_gate.shape[1])
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert out.dtype in (torch.bfloat16, torch.float32) and maps >= 1
    assert q.shape[1] >= n_heads * maps * head_dim and out.shape[1] >= n_heads * maps * value_dim and out.shape[0] >= q.shape[0]
    assert k_pages.shape[1:] == (n_kv_heads, PAGE, maps * head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert v_pages.shape == (k_pages.shape[0], n_kv_heads, PAGE, value_dim)
    if r1 is not None:
        assert r1.dtype == torch.float32 and r2.dtype == torch.float32 and r1.numel() == n_heads and r2.numel() == n_heads
    _check(_fn("attention_tc", "cml_attn_prefill_tc_maps")(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), k_pages.shape[0], _p(block_table),
        block_table.shape[1], _p(tile_seq), _p(tile_q0), n_tiles, _p(seq_row0), _p(seq_start), _p(seq_new), n_heads,
        n_kv_heads, head_dim, value_dim, rows_per_tile, heads_per_cta, head_chunks, int(window or 0), float(scale), _p(r1), _p(r2),
        int(chunk or 0), _p(sink), _p(head_gate), head_gate.stride(0) if head_gate is not None else 0, int(gate_col),
        int(maps), float(softcap or 0.0), 1 if out.dtype == torch.float32 else 0, int(keep_first or 0), _p(err), _stream()),
        "attn_prefill_tc")


def maps_difference(maps_out: torch.Tensor, lam: float, eps: float, out_scale: float, out: torch.Tensor, heads: int, value_dim: int):
    """out[r, head] = d / sqrt(mean(d^2) + eps) * out_scale with d = a1 - lam * a2 over the head's ``value_dim`` channels,
    from ``maps_out`` float32 [rows, heads * 2 * value_dim] (head by head: a1, a2), the two score maps' attentions."""
    _dev(maps_out, out)
    rows = maps_out.shape[0]
    assert maps_out.dtype == torch.float32 and maps_out.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == rows
    assert maps_out.shape[1] == heads * 2 * value_dim and out.shape[1] == heads * value_dim
    _check(_fn("attention_window", "cml_maps_difference")(
        _p(maps_out), maps_out.stride(0), _p(out), out.stride(0), dtype_code(out.dtype), rows, heads, value_dim, float(lam),
        float(eps), float(out_scale), _stream()), "maps_difference")


def gemm_tn_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int, group: int = 0, err=None, act=None):
    """c[M, N] (op)= a[M, K] @ w[N, K]^T with float accumulation on the CUDA cores.
    EPI_SWIGLU reads w as packed [2N, K] gate/up rows interleaved in groups of ``group``.
    ``err`` (int32[1]): set to 8 by the form that streams float weights through shared memory if one
    of its bounded waits runs out; by default this module's own word (``simt_error_word``)."""
    _dev(a, w, c)
    M, K = a.shape
    N = c.shape[1]
    assert c.shape[0] == M and w.shape[1] == K and a.dtype == w.dtype
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] == 2 * N and c.dtype == a.dtype
    else:
        assert w.shape[0] == N
        assert c.dtype == (a.dtype if epilogue == EPI_STORE else torch.float32)
    scratch = None
    if err is None:
        err = simt_error_word(a.device)
    if a.dtype == torch.float32 and M <= 64:      # the streaming form for few float rows: tickets and split sums
        f = _fn("gemm_simt", "cml_gemv_f32_scratch_bytes")
        f.restype = c_long
        scratch = zeroed_scratch(a.device, "gemv_f32", int(f(M, N, K, epilogue)))
    if epilogue == EPI_SWIGLU:
        _gate_act("gemm_simt", act)
    _check(_fn("gemm_simt", "cml_gemm_tn_simt")(_p(a), a.stride(0), _p(w), w.stride(0), _p(c), c.stride(0), M, N, K,
                                                dtype_code(a.dtype), epilogue, group, _p(scratch), _p(err), _stream()),
           "gemm_tn_simt")


def gemv_f32_partial_splits(a: torch.Tensor, w: torch.Tensor) -> int:
    """Ranges of K that ``gemv_f32_partial`` cuts a[M, K] @ w[N, K]^T into; 0 where it does not take
    the product (more than 64 rows, not float, sizes that do not allow 16-byte copies)."""
    if a.dtype != torch.float32 or w.dtype != torch.float32 or a.stride(1) != 1 or w.stride(1) != 1:
        return 0
    if (a.data_ptr() | w.data_ptr()) & 15:
        return 0
    return int(_fn("gemm_simt", "cml_gemv_f32_partial_splits")(a.shape[0], w.shape[0], a.shape[1], a.stride(0),
                                                               w.stride(0)))


def gemv_f32_partial(a: torch.Tensor, w: torch.Tensor, part: torch.Tensor, err: torch.Tensor):
    """part[r] = a @ w^T over range r of K (float, at most 64 rows): the product's sums left as
    partial sums for the kernel that reads them next, with no pass over them in between."""
    _dev(a, w, part, err)
    splits, M, N = part.shape
    assert part.dtype == torch.float32 and part.stride(2) == 1 and a.shape[0] == M and w.shape[0] == N
    _check(_fn("gemm_simt", "cml_gemv_f32_partial")(_p(a), a.stride(0), _p(w), w.stride(0), _p(part), part.stride(1),
                                                    part.stride(0), splits, M, N, a.shape[1], _p(err), _stream()),
           "gemv_f32_partial")


_scratch: dict = {}
_retired: list = []
_simt_err: dict = {}


def simt_error_word(device) -> torch.Tensor:
    """The error word ``gemm_tn_simt`` hands its kernels when the caller gives none."""
    key = torch.device(device)
    e = _simt_err.get(key)
    if e is None:
        e = torch.zeros(1, dtype=torch.int32, device=device)
        _simt_err[key] = e
    return e


def zeroed_scratch(device, name: str, n_bytes: int) -> torch.Tensor:
    """Device memory that kernels of this library leave zeroed between calls (tickets of
    the blocks of a kernel and the like); it only ever grows. Not to be made while a CUDA
    graph is being captured: the first call of a kernel that needs it should come before."""
    key = (torch.device(device), name)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n_bytes:
        if buf is not None:
            _retired.append(buf)               # captured graphs may still point at it
        buf = torch.zeros(max(n_bytes, 4096), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def argmax_rows(logits: torch.Tensor, out: torch.Tensor, err: torch.Tensor):
    """out[r] = index of the largest logit of row r, the lowest index among equals."""
    _dev(logits, out, err)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= rows
    scratch = zeroed_scratch(logits.device, "argmax", 16 * max(rows, 64))
    _check(_fn("sampling", "cml_argmax_rows")(_p(logits), logits.stride(0), rows, vocab, _p(out), _p(err), _p(scratch),
                                             _stream()), "argmax_rows")


def adjust_logits(logits: torch.Tensor, entries: torch.Tensor, biases: torch.Tensor, repeat_penalty: float,
                  presence_penalty: float, frequency_penalty: float):
    """entries: int32 [n, 3] of (row, token, count in history); biases: float32 [n]."""
    _dev(logits, entries, biases)
    n = entries.shape[0]
    assert entries.dtype == torch.int32 and entries.is_contiguous() and biases.dtype == torch.float32 and biases.numel() == n
    _check(_fn("sampling", "cml_adjust_logits")(_p(logits), logits.stride(0), logits.shape[1], _p(entries), _p(biases),
                                               n, float(repeat_penalty), float(presence_penalty),
                                               float(frequency_penalty), _stream()), "adjust_logits")


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float,
                draws: torch.Tensor, out: torch.Tensor, err: torch.Tensor, params=None):
    """One token per row of ``logits`` by the reference's stochastic sampler. ``params`` (float32 [4] on the
    device: temperature, top_k or 0, top_p or 1, min_p or 0), if given, is read by the kernel instead of
    the four arguments, so that a captured launch serves any values."""
    _dev(logits, draws, out, err, params)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and draws.dtype == torch.float32
    assert draws.numel() >= rows and out.dtype == torch.int32 and out.numel() >= rows
    _check(_fn("sampling", "cml_sample_rows")(_p(logits), logits.stride(0), rows, vocab, float(temperature),
                                             int(top_k or 0), float(top_p if top_p is not None else 1.0),
                                             float(min_p or 0.0), _p(params), _p(draws), _p(out), _p(err), _stream()),
           "sample_rows")


def adjust_dense(logits: torch.Tensor, counts: torch.Tensor, bias: torch.Tensor, penalties: torch.Tensor):
    """Bias and penalties from device-side state: ``counts`` int32 [rows, vocab] (how often a token
    stands in the row's history), ``bias`` float32 [vocab], ``penalties`` float32 [3] = repeat,
    presence, frequency. In place on ``logits`` (float32 [rows, vocab])."""
    _dev(logits, counts, bias, penalties)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and counts.dtype == torch.int32
    assert counts.shape == (rows, vocab) and counts.is_contiguous() and bias.numel() == vocab and penalties.numel() == 3
    assert bias.dtype == torch.float32 and penalties.dtype == torch.float32
    _check(_fn("sampling", "cml_adjust_dense")(_p(logits), logits.stride(0), rows, vocab, _p(counts), _p(bias),
                                              _p(penalties), _stream()), "adjust_dense")


def count_tokens(tokens: torch.Tensor, counts: torch.Tensor):
    """counts[r][tokens[r]] += 1 for the rows of ``counts`` (int32 [rows, vocab])."""
    _dev(tokens, counts)
    rows, vocab = counts.shape
    assert tokens.dtype == torch.int32 and tokens.numel() >= rows and counts.dtype == torch.int32 and counts.is_contiguous()
    _check(_fn("sampling", "cml_count_tokens")(_p(tokens), _p(counts), rows, vocab, _stream()), "count_tokens")


def draws_at(positions: torch.Tensor, seed: torch.Tensor, draws: torch.Tensor):
    """draws[r] = the draw of the stream of ``seed`` (int64 [1] on the device) for a history of
    positions[r] + 1 tokens: what ``sampling.options.unit_draw`` gives on the host."""
    _dev(positions, seed, draws)
    rows = draws.numel()
    assert positions.dtype == torch.int32 and positions.numel() >= rows and seed.dtype == torch.int64
    assert draws.dtype == torch.float32
    _check(_fn("sampling", "cml_draws_at")(_p(positions), _p(seed), _p(draws), rows, _stream()), "draws_at")


class NativeDecodeLoop:
    """The C++ decode loop (decode_loop.cu) bound to one captured step graph: ``run`` performs up
    to ``max_steps`` one-token steps (copy in, graph, sampling kernel, copy out) per call."""

    def __init__(self, n: int, layout, meta_dev: torch.Tensor, head_template, logits: torch.Tensor, err: torch.Tensor):
        import numpy as np
        dev = meta_dev.device
        size = _fn("sampling", "cml_decode_loop_size")()
        self._state = ctypes.create_string_buffer(size)
        self.n = n
        self.head_ints = layout.offsets["seq_start"][0] + n
        self.meta_host = torch.zeros(self.head_ints, dtype=torch.int32).pin_memory()
        self.meta_host.numpy()[:] = head_template[:self.head_ints]
        self.tokens_dev = torch.zeros(n, dtype=torch.int32, device=dev)
        self.tokens_host = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.draws_dev = torch.zeros(n, dtype=torch.float32, device=dev)
        self.draws_host = torch.zeros(n, dtype=torch.float32).pin_memory()
        self.scratch = zeroed_scratch(dev, "argmax", 16 * max(n, 64))
        self.logits, self.err, self.meta_dev = logits, err, meta_dev
        self._np = np
        _check(_fn("sampling", "cml_decode_loop_init")(
            ctypes.addressof(self._state), n, layout.offsets["tokens"][0], layout.offsets["row_pos"][0],
            layout.offsets["seq_slot"][0], layout.offsets["seq_start"][0], self.head_ints, _p(meta_dev), _p(self.meta_host), _p(logits),
            logits.stride(0), logits.shape[1], _p(self.tokens_dev), _p(self.tokens_host), _p(err), _p(self.scratch),
            _p(self.draws_dev), _p(self.draws_host)), "decode_loop_init", 0)
        self.h2d_bytes_per_step = self.head_ints * 4
        self.d2h_bytes_per_step = n * 4

    def run(self, graph_exec: int, tokens, positions, slots, history_lens, max_steps: int, stop_ids, temperature: float,
            top_k: int, top_p: float, min_p: float, seed: int, launches_per_step: int):
        np = self._np
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        slo = np.ascontiguousarray(slots, dtype=np.int32)
        assert tok.size == pos.size == slo.size == self.n
        hist = np.ascontiguousarray(history_lens, dtype=np.int32)
        stops = np.ascontiguousarray(list(stop_ids), dtype=np.int32)
        out = np.empty((max_steps, self.n), dtype=np.int32)
        done = ctypes.c_int(0)
        rc = _fn("sampling", "cml_decode_loop_run")(
            ctypes.addressof(self._state), graph_exec, _stream(), tok.ctypes.data, pos.ctypes.data, slo.ctypes.data,
            hist.ctypes.data,
            max_steps, stops.ctypes.data if stops.size else None, int(stops.size), float(temperature), int(top_k or 0),
            float(top_p if top_p is not None else 1.0), float(min_p or 0.0), int(seed or 0), out.ctypes.data,
            ctypes.addressof(done))
        _check(rc, "decode_loop_run", (launches_per_step + 1) * done.value)
        return out[:done.value], done.value


class FedDecodeLoop:
    """The C++ loop for a captured step graph that picks the greedy token itself and feeds it to
    the next step on the device: ``run`` queues all its steps at once and waits once."""
    RING = 256                  # steps one call can queue

    def __init__(self, n: int, layout, meta_dev: torch.Tensor, head_template):
        import numpy as np
        self._np = np
        self.n = n
        self.offsets = [layout.offsets[k][0] for k in ("tokens", "row_pos", "seq_slot", "seq_start")]
        self.head_ints = layout.offsets["seq_start"][0] + n
        self.meta_dev = meta_dev
        self.ring = torch.zeros((self.RING, self.head_ints), dtype=torch.int32).pin_memory()
        self.ring.numpy()[:] = head_template[:self.head_ints]
        self.out = torch.zeros((self.RING, n), dtype=torch.int32).pin_memory()
        self.h2d_bytes_per_step = (self.head_ints - n) * 4
        self.d2h_bytes_per_step = n * 4

    def run(self, graph_exec: int, tokens, positions, slots, steps: int, launches_per_step: int):
        np = self._np
        assert 1 <= steps <= self.RING
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        slo = np.ascontiguousarray(slots, dtype=np.int32)
        assert tok.size == pos.size == slo.size == self.n
        rc = _fn("sampling", "cml_decode_fed_run")(
            self.n, *self.offsets, self.head_ints, _p(self.meta_dev), self.ring.data_ptr(), graph_exec, _stream(),
            tok.ctypes.data, pos.ctypes.data, slo.ctypes.data, int(steps), self.out.data_ptr())
        _check(rc, "decode_fed_run", launches_per_step * steps)
        return self.out.numpy()[:steps].copy()
