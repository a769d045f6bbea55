"""ctypes view of include/ferrum_cuda.h: status codes, POD structs and the library loader.

The CUDA library is the only implementation of the hot path. If it cannot be loaded this module
raises; nothing in the package falls back to a CPU or PyTorch implementation.
"""
from __future__ import annotations

import ctypes as C
import os

FC_OK = 0
FC_ERR_SHAPE = -1
FC_ERR_RANGE = -2
FC_ERR_CONTEXT_FULL = -3
FC_ERR_OOM = -4
FC_ERR_DEVICE = -5
FC_ERR_INJECTED = -6
FC_ERR_TIMEOUT = -7
FC_ERR_ARG = -8
FC_ERR_UNSUPPORTED = -9

STATUS_NAMES = {
    FC_OK: "ok",
    FC_ERR_SHAPE: "bad shape",
    FC_ERR_RANGE: "index out of range",
    FC_ERR_CONTEXT_FULL: "context full",
    FC_ERR_OOM: "out of memory",
    FC_ERR_DEVICE: "device error",
    FC_ERR_INJECTED: "injected fault",
    FC_ERR_TIMEOUT: "timeout",
    FC_ERR_ARG: "bad argument",
    FC_ERR_UNSUPPORTED: "unsupported",
}

FC_F32, FC_Q8_0, FC_Q4_0, FC_F16, FC_FP8_E4M3, FC_FP8_E5M2, FC_MXFP4, FC_Q2_K = 0, 1, 2, 3, 4, 5, 6, 7
FC_ROPE_NORM, FC_ROPE_NEOX = 0, 1
FC_EXACT_F32, FC_TENSOR_F16 = 0, 1

f32p = C.POINTER(C.c_float)


class FcLlamaConfig(C.Structure):
    _fields_ = [
        ("vocab", C.c_uint32), ("ctx", C.c_uint32), ("dim", C.c_uint32), ("heads", C.c_uint32),
        ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("layers", C.c_uint32),
        ("hidden", C.c_uint32), ("rope_dim", C.c_uint32), ("rope_type", C.c_uint32),
        ("rope_base", C.c_float), ("eps", C.c_float), ("rope_linear_factor", C.c_float),
        ("n_freq_factors", C.c_uint32), ("freq_factors", f32p), ("tied", C.c_uint32),
    ]


LLAMA_BLOCK_FIELDS = ("attn_norm", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "ffn_norm", "gate",
                      "up", "down")


class FcLlamaBlock(C.Structure):
    _fields_ = [(n, f32p) for n in LLAMA_BLOCK_FIELDS]


class FcLlamaWeights(C.Structure):
    _fields_ = [("tok", f32p), ("blocks", C.POINTER(FcLlamaBlock)), ("out_norm", f32p),
                ("head", f32p)]


class FcGpt2Config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("vocab", "ctx", "dim", "heads", "layers", "hidden")]


GPT2_BLOCK_FIELDS = ("ln1_g", "ln1_b", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "ln2_g",
                     "ln2_b", "w1", "b1", "w2", "b2")


class FcGpt2Block(C.Structure):
    _fields_ = [(n, f32p) for n in GPT2_BLOCK_FIELDS]


class FcGpt2Weights(C.Structure):
    _fields_ = [("tok", f32p), ("pos", f32p), ("blocks", C.POINTER(FcGpt2Block)), ("lnf_g", f32p),
                ("lnf_b", f32p), ("head", f32p)]


class FcTensor(C.Structure):
    """One weight tensor: f32 `[in, out]` (kind FC_F32) or the tensor's GGUF block bytes (a block kind)."""
    _fields_ = [("data", C.c_void_p), ("kind", C.c_int)]


LLAMA_MATS = ("wq", "wk", "wv", "wo", "gate", "up", "down")
GPT2_MATS = ("wq", "wk", "wv", "wo", "w1", "w2")


class FcLlamaBlockT(C.Structure):
    _fields_ = [(n, FcTensor if n in LLAMA_MATS else f32p) for n in LLAMA_BLOCK_FIELDS]


class FcLlamaTensors(C.Structure):
    _fields_ = [("tok", FcTensor), ("blocks", C.POINTER(FcLlamaBlockT)), ("out_norm", f32p), ("head", FcTensor)]


class FcGpt2BlockT(C.Structure):
    _fields_ = [(n, FcTensor if n in GPT2_MATS else f32p) for n in GPT2_BLOCK_FIELDS]


class FcGpt2Tensors(C.Structure):
    _fields_ = [("tok", FcTensor), ("pos", f32p), ("blocks", C.POINTER(FcGpt2BlockT)), ("lnf_g", f32p), ("lnf_b", f32p),
                ("head", FcTensor)]


# Every symbol include/ferrum_cuda.h declares; tests check that the built library exports them.
EXPORTS = (
    "fc_device_open", "fc_device_close", "fc_device_name", "fc_device_props", "fc_last_error",
    "fc_device_stream", "fc_device_sync", "fc_device_launch_count", "fc_debug_fail_after",
    "fc_debug_profile", "fc_debug_profile_report", "fc_debug_matvec_kernel", "fc_debug_raise_status", "fc_debug_attention_f16",
    "fc_block_bytes", "fc_qweight_create", "fc_qweight_create_from_blocks", "fc_qweight_destroy",
    "fc_qweight_info", "fc_qweight_blocks", "fc_dequant", "fc_qmatmul", "fc_qmatmul_dev",
    "fc_qmatmul_dev_noalloc",
    "fc_llama_plan_bytes", "fc_gpt2_plan_bytes", "fc_llama_create", "fc_gpt2_create",
    "fc_llama_create_from_tensors", "fc_gpt2_create_from_tensors",
    "fc_model_destroy", "fc_model_pos", "fc_model_reset", "fc_model_info", "fc_model_feed",
    "fc_model_feed_batch", "fc_model_decode_greedy", "fc_model_topk", "fc_topk_dev", "fc_model_prefill", "fc_model_forward_all", "fc_model_score",
    "fc_model_score_dev", "fc_model_set_head_shard", "fc_model_trunk_dev",
    "fc_model_head_partial_dev", "fc_score_combine_dev",
    "fc_model_score_ragged", "fc_score_windows", "fc_model_token_logprobs",
    "fc_group_sequences", "fc_group_unique_id", "fc_group_create", "fc_group_destroy", "fc_group_score",
    "fc_group_last_exchange_ms",
)

LIB_NAME = "libferrum_cuda.so"


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


_lib = None


def load() -> C.CDLL:
    """Load libferrum_cuda.so (built in-tree by ferrum_gpu_b200.build) and set prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m ferrum_gpu_b200.build`. "
            "There is no CPU fallback for this path.")
    lib = C.CDLL(path)
    vp, u32, i32, u64, i64, sz = C.c_void_p, C.c_uint32, C.c_int32, C.c_uint64, C.c_int64, C.c_size_t
    P = C.POINTER
    sig = {
        "fc_device_open": (C.c_int, [C.c_int, P(vp)]),
        "fc_device_close": (C.c_int, [vp]),
        "fc_device_name": (C.c_int, [vp, C.c_char_p, sz]),
        "fc_device_props": (C.c_int, [vp, P(C.c_int), P(u64)]),
        "fc_last_error": (C.c_char_p, [vp]),
        "fc_device_stream": (vp, [vp]),
        "fc_device_sync": (C.c_int, [vp]),
        "fc_device_launch_count": (u64, [vp]),
        "fc_debug_fail_after": (C.c_int, [vp, i64]),
        "fc_debug_profile": (C.c_int, [vp, C.c_int]),
        "fc_debug_matvec_kernel": (C.c_int, [vp, C.c_int]),
        "fc_debug_raise_status": (C.c_int, [vp, C.c_int]),
        "fc_debug_profile_report": (C.c_int, [vp, C.c_char_p, sz]),
        "fc_model_topk": (C.c_int, [vp, u32, u32, C.c_float, vp, u32, vp, vp, P(u32)]),
        "fc_topk_dev": (C.c_int, [vp, vp, u32, u32, C.c_float, vp, u32, vp, vp, P(u32)]),
        "fc_debug_attention_f16": (C.c_int, [vp, vp, u32, u32, u32, u32, vp, C.c_int, C.c_int, P(C.c_float)]),
        "fc_block_bytes": (sz, [C.c_int, sz]),
        "fc_qweight_create": (C.c_int, [vp, C.c_int, vp, u32, u32, P(vp)]),
        "fc_qweight_create_from_blocks": (C.c_int, [vp, C.c_int, vp, sz, u32, u32, P(vp)]),
        "fc_qweight_destroy": (C.c_int, [vp]),
        "fc_qweight_info": (C.c_int, [vp, P(C.c_int), P(u32), P(u32), P(u64)]),
        "fc_qweight_blocks": (C.c_int, [vp, vp, sz]),
        "fc_dequant": (C.c_int, [vp, vp, sz]),
        "fc_qmatmul": (C.c_int, [vp, vp, u32, vp, C.c_int]),
        "fc_qmatmul_dev": (C.c_int, [vp, vp, u32, vp, C.c_int]),
        "fc_qmatmul_dev_noalloc": (C.c_int, [vp, vp, u32, vp]),
        "fc_llama_plan_bytes": (u64, [P(FcLlamaConfig), C.c_int, u32]),
        "fc_gpt2_plan_bytes": (u64, [P(FcGpt2Config), C.c_int, u32]),
        "fc_llama_create": (C.c_int, [vp, P(FcLlamaConfig), P(FcLlamaWeights), C.c_int, u32, u64, P(vp)]),
        "fc_gpt2_create": (C.c_int, [vp, P(FcGpt2Config), P(FcGpt2Weights), C.c_int, u32, u64, P(vp)]),
        "fc_llama_create_from_tensors": (C.c_int, [vp, P(FcLlamaConfig), P(FcLlamaTensors), C.c_int, u32, u64, P(vp)]),
        "fc_gpt2_create_from_tensors": (C.c_int, [vp, P(FcGpt2Config), P(FcGpt2Tensors), C.c_int, u32, u64, P(vp)]),
        "fc_model_destroy": (C.c_int, [vp]),
        "fc_model_pos": (C.c_int, [vp, u32, P(u32)]),
        "fc_model_reset": (C.c_int, [vp, u32]),
        "fc_model_info": (C.c_int, [vp, P(u32), P(u32), P(u32), P(C.c_int), P(u64)]),
        "fc_model_feed": (C.c_int, [vp, u32, i32, vp, P(i32)]),
        "fc_model_feed_batch": (C.c_int, [vp, u32, vp, vp, vp, vp]),
        "fc_model_decode_greedy": (C.c_int, [vp, u32, vp, vp, u32, vp]),
        "fc_model_prefill": (C.c_int, [vp, u32, vp, u32, vp, P(i32), C.c_int]),
        "fc_model_forward_all": (C.c_int, [vp, vp, u32, vp, C.c_int]),
        "fc_model_score": (C.c_int, [vp, vp, u32, u32, C.c_int, vp, vp, vp]),
        "fc_model_score_dev": (C.c_int, [vp, vp, u32, u32, C.c_int, vp, vp, vp]),
        "fc_model_set_head_shard": (C.c_int, [vp, u32, u32]),
        "fc_model_trunk_dev": (C.c_int, [vp, vp, u32, u32, C.c_int, vp]),
        "fc_model_head_partial_dev": (C.c_int, [vp, vp, vp, u32, C.c_int, vp]),
        "fc_score_combine_dev": (C.c_int, [vp, vp, u32, vp, u32, u32, vp, vp, vp]),
        "fc_model_score_ragged": (C.c_int, [vp, vp, vp, u32, C.c_int, vp, vp, vp]),
        "fc_score_windows": (u32, [u32, u32, u32, vp, vp, vp, u32]),
        "fc_model_token_logprobs": (C.c_int, [vp, vp, vp, vp, u32, C.c_int, vp, vp, vp]),
        "fc_group_sequences": (u32, [u32, u32, u32, vp, u32]),
        "fc_group_unique_id": (C.c_int, [vp, sz]),
        "fc_group_create": (C.c_int, [vp, vp, u32, u32, u32, vp, sz, P(vp)]),
        "fc_group_destroy": (C.c_int, [vp]),
        "fc_group_score": (C.c_int, [vp, vp, u32, u32, C.c_int, vp]),
        "fc_group_last_exchange_ms": (C.c_int, [vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
