"""ctypes binding of the C ABI declared in ``include/deers_b200.h``."""
from __future__ import annotations

import ctypes
import os

from .errors import CudaError

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libdeers_b200.so")

OK, ERR_NULL, ERR_SHAPE, ERR_DTYPE, ERR_LAYOUT, ERR_WORKSPACE, ERR_CUDA, ERR_KERNEL, ERR_UNSUPPORTED, ERR_DEVICE = range(10)
F16, F32 = 0, 1

# Every symbol include/deers_b200.h declares.
SYMBOLS = [
    "deers_b200_attn_desc_compact", "deers_b200_init", "deers_b200_destroy", "deers_b200_set_stream",
    "deers_b200_stream", "deers_b200_alloc", "deers_b200_free", "deers_b200_memcpy_h2d",
    "deers_b200_memcpy_d2h", "deers_b200_memcpy_d2d", "deers_b200_mem_info", "deers_b200_sync", "deers_b200_attn_workspace_bytes",
    "deers_b200_attn_fwd", "deers_b200_attn_bwd", "deers_b200_status_string", "deers_b200_last_error",
    "deers_b200_launch_count", "deers_b200_selftest_umma", "deers_b200_kernel_timing",
    "deers_b200_kernel_time", "deers_b200_attn_bwd_f16_static", "deers_b200_attn_host_scratch_bytes",
    "deers_b200_attn_fwd_bwd_host", "deers_b200_rope_pack",
    "deers_b200_optim_scratch_bytes", "deers_b200_grad_norm", "deers_b200_grad_clip", "deers_b200_adamw_step",
    "deers_b200_rmsnorm_fwd", "deers_b200_rmsnorm_bwd",
    "deers_b200_attn_decode_workspace_bytes", "deers_b200_attn_decode", "deers_b200_gemm_f16",
    "deers_b200_gemm_f32_workspace_bytes", "deers_b200_gemm_f32", "deers_b200_rmsnorm_bwd_add",
    "deers_b200_embedding_fwd", "deers_b200_embedding_bwd", "deers_b200_cross_entropy_scratch_bytes",
    "deers_b200_cross_entropy_fwd", "deers_b200_cross_entropy_bwd",
    "deers_b200_gpt_create", "deers_b200_gpt_destroy", "deers_b200_gpt_num_params", "deers_b200_gpt_param_info",
    "deers_b200_gpt_param_set", "deers_b200_gpt_param_get", "deers_b200_gpt_set_graph", "deers_b200_gpt_graph_active",
    "deers_b200_gpt_forward",
    "deers_b200_gpt_forward_backward", "deers_b200_gpt_train_step", "deers_b200_gpt_train_step_host",
    "deers_b200_shard_range", "deers_b200_comm_init_all", "deers_b200_comm_export", "deers_b200_comm_init_ipc",
    "deers_b200_comm_destroy", "deers_b200_comm_set_lanes", "deers_b200_allgather_o", "deers_b200_allgather_join", "deers_b200_allgather_flush",
    "deers_b200_selftest_wait", "deers_b200_split_f16x3", "deers_b200_gemm_f16x3_workspace_bytes", "deers_b200_gemm_f16x3",
]
IPC_HANDLE_BYTES = 72
K_FWD, K_BWD_PREP, K_BWD_MAIN, K_BWD_DQ, K_ROPE, K_OPTIM, K_NORM, K_DECODE, K_GEMM, K_GPT, K_GEMM_X3 = range(11)
EPI_NONE, EPI_ADD, EPI_RELU_SQ, EPI_MUL_AUX2 = range(4)


class AttnDesc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("H", ctypes.c_int32), ("T", ctypes.c_int32), ("D", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("causal", ctypes.c_int32), ("scale", ctypes.c_float),
                ("q_strides", ctypes.c_int64 * 4), ("k_strides", ctypes.c_int64 * 4),
                ("v_strides", ctypes.c_int64 * 4), ("o_strides", ctypes.c_int64 * 4),
                ("do_strides", ctypes.c_int64 * 4), ("dq_strides", ctypes.c_int64 * 4),
                ("dk_strides", ctypes.c_int64 * 4), ("dv_strides", ctypes.c_int64 * 4)]


class RopeDesc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32), ("D", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("inverse", ctypes.c_int32),
                ("src_strides", ctypes.c_int64 * 4), ("dst_strides", ctypes.c_int64 * 4)]


class OptimTensor(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("g", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("n", ctypes.c_int64)]


class AdamWHyper(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_double), ("beta1", ctypes.c_double), ("beta2", ctypes.c_double),
                ("eps", ctypes.c_double), ("weight_decay", ctypes.c_double), ("step", ctypes.c_int64)]


class DecodeDesc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Tq", ctypes.c_int32), ("Tk", ctypes.c_int32),
                ("D", ctypes.c_int32), ("dtype", ctypes.c_int32), ("causal", ctypes.c_int32), ("scale", ctypes.c_float),
                ("q_strides", ctypes.c_int64 * 4), ("k_strides", ctypes.c_int64 * 4),
                ("v_strides", ctypes.c_int64 * 4), ("o_strides", ctypes.c_int64 * 4)]


class GemmEpilogue(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("residual", ctypes.c_void_p), ("ld_residual", ctypes.c_int64),
                ("aux", ctypes.c_void_p)]


class GptConfig(ctypes.Structure):
    _fields_ = [("vocab_size", ctypes.c_int32), ("sequence_len", ctypes.c_int32), ("n_layer", ctypes.c_int32),
                ("n_head", ctypes.c_int32), ("n_embd", ctypes.c_int32), ("mlp_hidden_dim", ctypes.c_int32),
                ("rms_norm_eps", ctypes.c_double), ("rope_base", ctypes.c_float)]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the shared library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python -m deers_b200.build` "
                          "(the attention path has no CPU or PyTorch fallback)")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    dp = ctypes.POINTER(AttnDesc)
    L.deers_b200_attn_desc_compact.argtypes = [dp, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                               ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_float]
    L.deers_b200_attn_desc_compact.restype = None
    L.deers_b200_init.argtypes = [i32, vp, ctypes.POINTER(vp)]
    L.deers_b200_destroy.argtypes = [vp]
    L.deers_b200_destroy.restype = None
    L.deers_b200_set_stream.argtypes = [vp, vp]
    L.deers_b200_stream.argtypes = [vp]
    L.deers_b200_stream.restype = vp
    L.deers_b200_alloc.argtypes = [vp, sz, ctypes.POINTER(vp)]
    L.deers_b200_free.argtypes = [vp, vp]
    for n in ("h2d", "d2h", "d2d"):
        getattr(L, f"deers_b200_memcpy_{n}").argtypes = [vp, vp, vp, sz]
    L.deers_b200_sync.argtypes = [vp]
    L.deers_b200_mem_info.argtypes = [vp, ctypes.POINTER(sz), ctypes.POINTER(sz)]
    L.deers_b200_attn_workspace_bytes.argtypes = [dp, i32]
    L.deers_b200_attn_workspace_bytes.restype = sz
    L.deers_b200_attn_fwd.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp, sz]
    L.deers_b200_attn_bwd.argtypes = [vp, dp] + [vp] * 10 + [sz]
    L.deers_b200_attn_bwd_f16_static.argtypes = [vp, dp] + [vp] * 9
    L.deers_b200_attn_host_scratch_bytes.argtypes = [dp, i32]
    L.deers_b200_attn_host_scratch_bytes.restype = sz
    L.deers_b200_attn_fwd_bwd_host.argtypes = [vp, dp] + [vp] * 9 + [i32, vp, sz]
    L.deers_b200_rope_pack.argtypes = [vp, ctypes.POINTER(RopeDesc), vp, vp, vp, vp]
    tp = ctypes.POINTER(OptimTensor)
    L.deers_b200_optim_scratch_bytes.argtypes = []
    L.deers_b200_optim_scratch_bytes.restype = sz
    L.deers_b200_grad_norm.argtypes = [vp, i32, tp, vp, vp, sz]
    L.deers_b200_grad_clip.argtypes = [vp, i32, tp, vp, ctypes.c_double]
    L.deers_b200_adamw_step.argtypes = [vp, i32, tp, ctypes.POINTER(AdamWHyper), vp, ctypes.c_double]
    L.deers_b200_rmsnorm_fwd.argtypes = [vp, ctypes.c_int64, ctypes.c_int32, ctypes.c_double, vp, vp, vp]
    L.deers_b200_rmsnorm_bwd.argtypes = [vp, ctypes.c_int64, ctypes.c_int32, vp, vp, vp, vp]
    ddp = ctypes.POINTER(DecodeDesc)
    L.deers_b200_attn_decode_workspace_bytes.argtypes = [ddp]
    L.deers_b200_attn_decode_workspace_bytes.restype = sz
    L.deers_b200_attn_decode.argtypes = [vp, ddp, vp, vp, vp, vp, vp, vp, sz]
    i64 = ctypes.c_int64
    L.deers_b200_gemm_f16.argtypes = [vp, i32, i32, i32, vp, i64, i32, vp, i64, i32, vp, i64]
    L.deers_b200_gemm_f32_workspace_bytes.argtypes = [vp, i32, i32, i32]
    L.deers_b200_gemm_f32_workspace_bytes.restype = sz
    L.deers_b200_gemm_f32.argtypes = [vp, i32, i32, i32, vp, i64, i32, vp, i64, i32, vp, i64,
                                      ctypes.POINTER(GemmEpilogue), vp, sz]
    L.deers_b200_split_f16x3.argtypes = [vp, i64, ctypes.c_int32, vp, i64, ctypes.c_float, vp, vp, i64]
    L.deers_b200_gemm_f16x3_workspace_bytes.argtypes = [vp, i32, i32, i32]
    L.deers_b200_gemm_f16x3_workspace_bytes.restype = sz
    L.deers_b200_gemm_f16x3.argtypes = [vp, i32, i32, i32, vp, vp, i64, i32, vp, vp, i64, i32, vp, i64, ctypes.c_float, vp, sz]
    L.deers_b200_rmsnorm_bwd_add.argtypes = [vp, i64, ctypes.c_int32, vp, vp, vp, vp, vp]
    L.deers_b200_embedding_fwd.argtypes = [vp, vp, vp, i64, ctypes.c_int32, i64, vp]
    L.deers_b200_embedding_bwd.argtypes = [vp, vp, vp, i64, ctypes.c_int32, i64, vp]
    L.deers_b200_cross_entropy_scratch_bytes.argtypes = [i64]
    L.deers_b200_cross_entropy_scratch_bytes.restype = sz
    L.deers_b200_cross_entropy_fwd.argtypes = [vp, i64, i64, vp, i64, vp, vp, vp, vp, sz]
    L.deers_b200_cross_entropy_bwd.argtypes = [vp, i64, i64, vp, i64, vp, vp, ctypes.c_float, vp, i64]
    gcp, hp = ctypes.POINTER(GptConfig), ctypes.POINTER(AdamWHyper)
    L.deers_b200_gpt_create.argtypes = [vp, gcp, ctypes.c_int32, ctypes.POINTER(vp)]
    L.deers_b200_gpt_destroy.argtypes = [vp]
    L.deers_b200_gpt_destroy.restype = None
    L.deers_b200_gpt_num_params.argtypes = [vp]
    L.deers_b200_gpt_param_info.argtypes = [vp, i32, ctypes.c_char_p, sz, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    L.deers_b200_gpt_param_set.argtypes = [vp, i32, i32, vp]
    L.deers_b200_gpt_param_get.argtypes = [vp, i32, i32, vp]
    L.deers_b200_gpt_set_graph.argtypes = [vp, i32]
    L.deers_b200_gpt_graph_active.argtypes = [vp]
    L.deers_b200_gpt_forward.argtypes = [vp, vp, ctypes.c_int32, ctypes.c_int32, vp]
    L.deers_b200_gpt_forward_backward.argtypes = [vp, vp, vp, ctypes.c_int32, ctypes.c_int32, vp]
    L.deers_b200_gpt_train_step.argtypes = [vp, vp, vp, ctypes.c_int32, ctypes.c_int32, hp, ctypes.c_double, vp, vp]
    L.deers_b200_gpt_train_step_host.argtypes = [vp, vp, vp, ctypes.c_int32, ctypes.c_int32, hp, ctypes.c_double,
                                                 ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float)]
    L.deers_b200_shard_range.argtypes = [i64, ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    L.deers_b200_shard_range.restype = None
    L.deers_b200_comm_init_all.argtypes = [ctypes.c_int32, ctypes.POINTER(vp), ctypes.POINTER(vp), sz, ctypes.POINTER(vp)]
    L.deers_b200_comm_export.argtypes = [vp, vp, ctypes.c_char_p]
    L.deers_b200_comm_init_ipc.argtypes = [vp, ctypes.c_int32, ctypes.c_int32, vp, sz, ctypes.c_char_p, ctypes.POINTER(vp)]
    L.deers_b200_comm_destroy.argtypes = [vp]
    L.deers_b200_comm_destroy.restype = None
    L.deers_b200_allgather_o.argtypes = [vp, sz, sz]
    L.deers_b200_comm_set_lanes.argtypes = [vp, i32]
    L.deers_b200_allgather_join.argtypes = [vp]
    L.deers_b200_allgather_flush.argtypes = [vp]
    L.deers_b200_status_string.argtypes = [i32]
    L.deers_b200_status_string.restype = ctypes.c_char_p
    L.deers_b200_last_error.argtypes = [vp]
    L.deers_b200_last_error.restype = ctypes.c_char_p
    L.deers_b200_launch_count.argtypes = [vp]
    L.deers_b200_launch_count.restype = ctypes.c_uint64
    L.deers_b200_selftest_umma.argtypes = [vp, ctypes.POINTER(ctypes.c_float)]
    L.deers_b200_selftest_wait.argtypes = [vp, ctypes.c_uint32, ctypes.POINTER(ctypes.c_int32)]
    L.deers_b200_kernel_timing.argtypes = [vp, i32]
    L.deers_b200_kernel_time.argtypes = [vp, i32, i32, ctypes.POINTER(ctypes.c_double),
                                         ctypes.POINTER(ctypes.c_uint64)]
    _lib = L
    return L


def status_string(status: int) -> str:
    return lib().deers_b200_status_string(status).decode()


def check(status: int, ctx=None) -> None:
    """Maps a non-zero status to CudaError, like Error::Cuda(String) on the deers side."""
    if status != OK:
        text = status_string(status)
        if ctx is not None:
            detail = lib().deers_b200_last_error(ctx).decode()
            if detail:
                text = f"{text} [{detail}]"
        raise CudaError(status, text)
