"""ctypes view of the C ABI in include/b200_kquant.h.

The shared library is the product: importing this module fails loudly if it has not been built,
and nothing here computes on the CPU.  torch is used only to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.environ.get("B200_KQ_LIB") or os.path.join(_HERE, "libb200kq.so")

TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K, TYPE_I32 = 0, 1, 2, 8, 12, 14, 26

OK = 0
STATUS_NAMES = {0: "OK", -1: "INVALID", -2: "ALLOC", -3: "CUDA", -4: "UNSUPPORTED", -5: "BOUNDS",
                -6: "TIMEOUT", -7: "STATE"}


class B200Error(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"b200 status {STATUS_NAMES.get(status, status)}: {msg}")
        self.status = status


class Tensor(C.Structure):
    """b200_tensor: the 296-byte packed descriptor (wire form of ggml's rpc_tensor)."""
    _pack_ = 1
    _fields_ = [
        ("id", C.c_uint64), ("type", C.c_uint32), ("buffer", C.c_uint64),
        ("ne", C.c_uint32 * 4), ("nb", C.c_uint32 * 4), ("op", C.c_uint32),
        ("op_params", C.c_int32 * 16), ("flags", C.c_int32), ("src", C.c_uint64 * 10),
        ("view_src", C.c_uint64), ("view_offs", C.c_uint64), ("data", C.c_uint64),
        ("name", C.c_char * 64), ("padding", C.c_char * 4),
    ]


class StageConfig(C.Structure):
    _fields_ = [
        ("n_layer", C.c_int32), ("layer_begin", C.c_int32), ("layer_end", C.c_int32),
        ("n_embd", C.c_int32), ("n_head", C.c_int32), ("n_head_kv", C.c_int32),
        ("head_dim", C.c_int32), ("n_ff", C.c_int32), ("n_vocab", C.c_int32),
        ("n_expert", C.c_int32), ("n_expert_used", C.c_int32), ("n_ff_exp", C.c_int32),
        ("n_ctx", C.c_int32), ("n_seq", C.c_int32),
        ("rope_neox", C.c_int32), ("qkv_bias", C.c_int32), ("qk_norm", C.c_int32),
        ("has_embd", C.c_int32), ("has_output", C.c_int32),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float),
        ("n_ubatch", C.c_int32), ("device", C.c_int32),
        ("kv_type_k", C.c_int32), ("kv_type_v", C.c_int32),
    ]


class GgufMeta(C.Structure):
    _fields_ = [
        ("architecture", C.c_char * 64), ("tokenizer_model", C.c_char * 64),
        ("context_length", C.c_uint32), ("vocab_size", C.c_uint32), ("embedding_length", C.c_uint32),
        ("head_count", C.c_uint32), ("head_count_kv", C.c_uint32), ("block_count", C.c_uint32),
        ("feed_forward_length", C.c_uint32), ("key_length", C.c_uint32), ("value_length", C.c_uint32),
        ("expert_count", C.c_uint32), ("expert_used_count", C.c_uint32),
        ("expert_feed_forward_length", C.c_uint32),
        ("rope_freq_base", C.c_float), ("rope_scale", C.c_float), ("rms_epsilon", C.c_float),
    ]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("type", C.c_uint32), ("n_dims", C.c_uint32), ("ne", C.c_int64 * 4),
                ("file_offset", C.c_uint64), ("nbytes", C.c_uint64)]


class GgufByteProfile(C.Structure):
    _fields_ = [("expert_count", C.c_uint32), ("expert_used_count", C.c_uint32),
                ("full_model_bytes", C.c_uint64), ("base_resident_bytes", C.c_uint64),
                ("expert_tensor_bytes", C.c_uint64), ("file_overhead_bytes", C.c_uint64)]


_lib = None

vp, i64, i32, u32, u64, sz = C.c_void_p, C.c_int64, C.c_int32, C.c_uint32, C.c_uint64, C.c_size_t

# name -> (restype, argtypes); every symbol include/b200_kquant.h declares
SIGNATURES = {
    "b200_status_string": (C.c_char_p, [i32]),
    "b200_last_error": (C.c_char_p, []),
    "b200_check_device_waits": (i32, []),
    "b200_reg_name": (C.c_char_p, []),
    "b200_reg_device_count": (i32, []),
    "b200_dev_name": (i32, [i32, C.c_char_p, sz]),
    "b200_dev_description": (i32, [i32, C.c_char_p, sz]),
    "b200_dev_memory": (i32, [i32, C.POINTER(sz), C.POINTER(sz)]),
    "b200_dev_supports_op": (i32, [u32, u32, u32]),
    "b200_buft_alignment": (sz, []),
    "b200_buft_max_size": (sz, [i32]),
    "b200_buft_alloc_size": (sz, [u32, C.POINTER(u32 * 4)]),
    "b200_buffer_alloc": (i32, [i32, sz, C.POINTER(vp)]),
    "b200_buffer_free": (None, [vp]),
    "b200_buffer_get_base": (vp, [vp]),
    "b200_buffer_get_size": (sz, [vp]),
    "b200_buffer_get_device": (i32, [vp]),
    "b200_buffer_clear": (i32, [vp, C.c_uint8]),
    "b200_buffer_init_tensor": (i32, [vp, C.POINTER(Tensor)]),
    "b200_buffer_set_tensor": (i32, [vp, C.POINTER(Tensor), vp, sz, sz]),
    "b200_buffer_get_tensor": (i32, [vp, C.POINTER(Tensor), vp, sz, sz]),
    "b200_buffer_cpy_tensor": (i32, [C.POINTER(Tensor), C.POINTER(Tensor), sz, sz]),
    "b200_backend_init": (i32, [i32, C.POINTER(vp)]),
    "b200_backend_free": (None, [vp]),
    "b200_backend_graph_compute": (i32, [vp, C.POINTER(u64), u32, C.POINTER(Tensor), u32]),
    "b200_backend_synchronize": (i32, [vp]),
    "b200_backend_stream": (vp, [vp]),
    "b200_row_bytes": (sz, [u32, i64]),
    "b200_device_row_bytes": (sz, [u32, i64]),
    "b200_repack_q6k": (i32, [vp, vp, i64, i64, vp]),
    "b200_unpack_q6k": (i32, [vp, vp, i64, i64, vp]),
    "b200_quantize_act": (i32, [vp, i64, i64, vp, vp, vp, vp]),
    "b200_mul_mat_scratch_bytes": (sz, [i64, i64]),
    "b200_mul_mat": (i32, [u32, vp, vp, i64, i64, i64, vp, vp, sz, vp]),
    "b200_mul_mat_q8": (i32, [u32, vp, vp, vp, vp, i64, i64, i64, vp, vp, vp, vp]),
    "b200_mul_mat_static": (i32, [u32, vp, vp, i64, i64, i64, vp, vp]),
    "b200_probe_int8_mma": (i32, [i32, i32, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "b200_block_sums": (i32, [u32, vp, vp, vp, i64, i64, i64, vp, vp, vp]),
    "b200_rms_norm": (i32, [vp, vp, i64, i64, C.c_float, vp, vp]),
    "b200_rope": (i32, [vp, vp, i64, i64, i64, C.c_float, i32, vp]),
    "b200_swiglu": (i32, [vp, vp, i64, vp, vp]),
    "b200_add": (i32, [vp, vp, i64, vp, vp]),
    "b200_add_bias": (i32, [vp, vp, i64, i64, vp]),
    "b200_cpy_f32_f16": (i32, [vp, i64, vp, vp]),
    "b200_attention": (i32, [vp, vp, vp, i64, i64, i64, i64, i64, vp, vp, sz, vp]),
    "b200_attention_scratch_bytes": (sz, [i64, i64, i64, i64]),
    "b200_handoff_create": (i32, [sz, i32, C.POINTER(vp)]),
    "b200_handoff_export": (i32, [vp, vp]),
    "b200_handoff_open": (i32, [vp, sz, i32, C.POINTER(vp)]),
    "b200_handoff_open_local": (i32, [vp, C.POINTER(vp)]),
    "b200_handoff_send": (i32, [vp, vp, sz, u64, u64, vp]),
    "b200_handoff_wait": (i32, [vp, vp, sz, u64, u64, C.POINTER(vp), vp]),
    "b200_handoff_release": (i32, [vp, u64, vp]),
    "b200_handoff_status": (i32, [vp, C.POINTER(i32)]),
    "b200_handoff_free": (None, [vp]),
    "b200_kv_row_bytes": (sz, [u32, i64]),
    "b200_kv_types_for_model_bytes": (None, [u64, C.POINTER(u32), C.POINTER(u32)]),
    "b200_kv_store": (i32, [vp, vp, vp, i64, i64, i64, C.c_float, i32, u32, u32, vp, vp, vp]),
    "b200_attention_kv": (i32, [vp, vp, vp, u32, u32, i64, i64, i64, i64, i64, vp, vp, sz, vp]),
    "b200_get_rows": (i32, [u32, vp, vp, i64, i64, vp, vp]),
    "b200_argmax": (i32, [vp, i64, i64, vp, vp]),
    "b200_mul_mat_id_scratch_bytes": (sz, [i64, i64, i64, i64]),
    "b200_mul_mat_id": (i32, [u32, vp, i64, vp, i64, vp, i64, i64, i64, vp, vp, sz, vp]),
    "b200_moe_route": (i32, [vp, i64, i64, i64, vp, vp, vp]),
    "b200_moe_route_masked": (i32, [vp, i64, i64, i64, vp, vp, vp, vp]),
    "b200_logit_signals_scratch_bytes": (sz, [i64]),
    "b200_logit_signals": (i32, [vp, i64, i64, vp, vp, vp, vp, sz, vp]),
    "b200_stage_create": (i32, [C.POINTER(StageConfig), C.POINTER(vp)]),
    "b200_stage_free": (None, [vp]),
    "b200_stage_set_tensor": (i32, [vp, C.c_char_p, u32, vp, sz]),
    "b200_stage_get_tensor": (i32, [vp, C.c_char_p, vp, sz]),
    "b200_stage_generate": (i32, [vp, u64]),
    "b200_stage_weight_bytes": (sz, [vp]),
    "b200_stage_forward": (i32, [vp, vp, vp, i32, i32, i32, i32, vp, vp, i32, vp, vp]),
    "b200_stage_profile_decode": (i32, [vp, i32, i32, u32, i32, C.POINTER(C.c_float), C.POINTER(i64)]),
    "b200_stage_tensor_count": (i64, [vp]),
    "b200_stage_tensor_info": (i32, [vp, i64, C.c_char_p, sz, C.POINTER(u32), C.POINTER(i64 * 3)]),
    "b200_gguf_open": (i32, [C.c_char_p, C.POINTER(vp)]),
    "b200_gguf_close": (None, [vp]),
    "b200_gguf_get_meta": (i32, [vp, C.POINTER(GgufMeta)]),
    "b200_gguf_tensor_count": (i64, [vp]),
    "b200_gguf_tensor_info": (i32, [vp, i64, C.POINTER(GgufTensor)]),
    "b200_gguf_find_tensor": (i64, [vp, C.c_char_p]),
    "b200_gguf_read_tensor": (i32, [vp, i64, vp, sz]),
    "b200_gguf_byte_profile": (i32, [vp, C.POINTER(GgufByteProfile)]),
    "b200_gguf_stage_config": (i32, [vp, i32, i32, i32, i32, i32, i32, C.POINTER(StageConfig)]),
    "b200_stage_load_gguf": (i32, [vp, vp, C.POINTER(i64), C.POINTER(i64)]),
    "b200_rpc_server_start": (i32, [C.c_char_p, i32, C.c_char_p, C.POINTER(vp)]),
    "b200_rpc_server_port": (i32, [vp]),
    "b200_rpc_server_stop": (None, [vp]),
    "b200_moe_assign": (i32, [vp, i32, i32, i32, i32, i32, i32, vp, i32, C.POINTER(i32), C.POINTER(i32),
                              C.POINTER(i32)]),
    "b200_gguf_write_expert_shard": (i32, [vp, vp, i32, C.c_char_p, C.POINTER(u64)]),
    "b200_stage_set_expert_mask": (i32, [vp, vp, i32]),
    "b200_stage_peek": (i32, [vp, C.c_char_p, vp, C.c_size_t]),
    "b200_stage_synchronize": (i32, [vp]),
    "b200_stage_kernel_launches": (i64, [vp]),
}


def lib():
    """Load libb200kq.so; raises if the CUDA library has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -m mesh_llm_b200.build` "
                "(there is no CPU fallback)")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            if not hasattr(L, name):
                continue  # reported by the symbol test; calling it raises AttributeError
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status):
    if status != OK:
        raise B200Error(status, lib().b200_last_error().decode(errors="replace"))


def ptr(t):
    """device (or host) address of a torch tensor / numpy array / int / None"""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def cur_stream():
    import torch

    return torch.cuda.current_stream().cuda_stream
