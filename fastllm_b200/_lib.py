"""ctypes binding of the C ABI in include/fastllm_b200.h.

This is the Python twin of the cgo/FFI stub a maintainer of the reference would add (INTEGRATION.md shows the Rust
one).  There is no fallback: if libfastllm_b200.so is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfastllm_b200.so")

FL_ARCH = {"llama": 0, "mistral": 1, "qwen2": 2, "mixtral": 3, "bert": 4, "nifunex": 5, "rofetar": 6, "tozarax": 7, "medulorn": 8}
FL_MIXER = {"gla": 0, "latent_attention": 1, "attention": 2, "mamba2": 3, "delta": 4, "lightning": 5}
FL_ACT = {"swish_clamp": 0, "gelu_tanh": 1, "relu2": 2, "relu": 3}
FL_ROT_SCALE = {"yarn": 0, "bands": 1}
FL_ROUTER = {"softmax": 0, "sigmoid_groups": 1}
FL_FFN = {"none": 0, "dense": 1, "moe": 2}
FL_DTYPE_F32, FL_DTYPE_BF16, FL_DTYPE_F16 = 0, 1, 2


class FlConfig(C.Structure):
    _fields_ = [("arch", C.c_int32), ("hidden_size", C.c_int32), ("intermediate_size", C.c_int32),
                ("vocab_size", C.c_int32), ("num_hidden_layers", C.c_int32), ("num_attention_heads", C.c_int32),
                ("num_key_value_heads", C.c_int32), ("max_position_embeddings", C.c_int32),
                ("sliding_window", C.c_int32), ("qkv_bias", C.c_int32), ("num_local_experts", C.c_int32),
                ("num_experts_per_tok", C.c_int32), ("norm_eps", C.c_float), ("rope_theta", C.c_double),
                ("tp_rank", C.c_int32), ("tp_size", C.c_int32), ("ep_dp_attention", C.c_int32), ("reserved", C.c_int32 * 5)]


class FlLayerDesc(C.Structure):
    """fl_layer_desc: one layer of a layered model (mixer + feed-forward, every size and constant)."""
    _fields_ = [("mixer", C.c_int32), ("heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("decay_rank", C.c_int32),
                ("tau", C.c_float), ("rot_dim", C.c_int32), ("kv_rank", C.c_int32), ("kv_from", C.c_int32), ("window", C.c_int32),
                ("rot_dims", C.c_int32), ("rot_base", C.c_double), ("scale", C.c_float), ("yarn_factor", C.c_float),
                ("yarn_original", C.c_float), ("yarn_fast", C.c_float), ("yarn_slow", C.c_float), ("ffn", C.c_int32), ("ff", C.c_int32),
                ("limit", C.c_float), ("experts", C.c_int32), ("top", C.c_int32), ("shared_ff", C.c_int32), ("shared_limit", C.c_float),
                ("kv_heads", C.c_int32), ("conv", C.c_int32), ("state", C.c_int32), ("groups", C.c_int32), ("norm_groups", C.c_int32),
                ("softcap", C.c_float), ("sink", C.c_int32), ("rot_halves", C.c_int32), ("ffn_act", C.c_int32), ("ffn_bias", C.c_int32),
                ("no_qk_norm", C.c_int32), ("beside", C.c_int32), ("router", C.c_int32), ("route_groups", C.c_int32),
                ("route_keep", C.c_int32), ("qkv_bias", C.c_int32), ("qk_norm_whole", C.c_int32), ("mask_chunk", C.c_int32),
                ("keep_first", C.c_int32), ("rot_scaling", C.c_int32), ("out_scale", C.c_float), ("pair_sum", C.c_int32),
                ("router_bias", C.c_int32), ("shared_plain", C.c_int32), ("reserved", C.c_int32 * 2)]


class FlStackConfig(C.Structure):
    _fields_ = [("arch", C.c_int32), ("vocab", C.c_int32), ("width", C.c_int32), ("n_layers", C.c_int32), ("norm_eps", C.c_float),
                ("compute_dtype", C.c_int32), ("norm_plain", C.c_int32), ("no_pre_norm", C.c_int32), ("no_post_norm", C.c_int32),
                ("max_positions", C.c_int32), ("canon_taps", C.c_int32), ("gated_residual", C.c_int32), ("depth_avg", C.c_int32),
                ("post_sum_norm", C.c_int32), ("residual_alpha", C.c_float), ("norm_scalar", C.c_int32), ("embed_scale", C.c_float),
                ("logit_softcap", C.c_float), ("token_shift", C.c_int32), ("reserved", C.c_int32 * 3)]


class FastllmError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"fastllm_b200 error {code}: {msg}")
        self.code = code


# every symbol include/fastllm_b200.h declares: name -> (restype, argtypes)
_VP, _I, _U64, _SZ = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t
SYMBOLS = {
    "fl_init": (_I, [_I]),
    "fl_last_error": (C.c_char_p, []),
    "fl_version": (_I, []),
    "fl_device_synchronize": (_I, []),
    "fl_model_create": (_I, [C.POINTER(FlConfig), C.POINTER(_VP)]),
    "fl_model_create_layered": (_I, [C.POINTER(FlStackConfig), C.POINTER(FlLayerDesc), C.POINTER(_VP)]),
    "fl_cache_create_pooled": (_I, [_VP, _I, _I, _I, C.POINTER(_VP)]),
    "fl_cache_pool_stats": (_I, [_VP, C.POINTER(_I), C.POINTER(_I)]),
    "fl_forward_ragged": (_I, [_VP, _VP, _VP, _VP, _I, _VP, _VP, _I, _VP]),
    "fl_model_put_tensor": (_I, [_VP, C.c_char_p, _I, C.POINTER(C.c_int64), _I, _VP]),
    "fl_model_random_init": (_I, [_VP, _U64, C.c_float]),
    "fl_model_finalize": (_I, [_VP]),
    "fl_model_clone": (_I, [_VP, C.POINTER(_VP)]),
    "fl_model_destroy": (_I, [_VP]),
    "fl_model_weight_bytes": (_I, [_VP, C.POINTER(_U64)]),
    "fl_cache_create": (_I, [_VP, _I, _I, C.POINTER(_VP)]),
    "fl_cache_reset": (_I, [_VP]),
    "fl_cache_kv_len": (_I, [_VP, C.POINTER(_I)]),
    "fl_cache_fill_synthetic": (_I, [_VP, _I, _I, _U64]),
    "fl_cache_destroy": (_I, [_VP]),
    "fl_forward": (_I, [_VP, _VP, _VP, _I, _I, _SZ, _VP]),
    "fl_forward_greedy": (_I, [_VP, _VP, _VP, _I, _I, _SZ, _VP]),
    "fl_decode_greedy_loop": (_I, [_VP, _VP, _VP, _I, _SZ, _I, _VP, C.POINTER(C.c_float)]),
    "fl_sampler_create": (_I, [_U64, C.c_double, C.POINTER(_VP)]),
    "fl_sampler_sample": (_I, [_VP, _VP, _SZ, C.POINTER(C.c_uint32)]),
    "fl_argmax_rows": (_I, [_VP, _I, _SZ, _VP]),
    "fl_sampler_next_u32": (_I, [_VP, C.POINTER(C.c_uint32)]),
    "fl_sampler_destroy": (_I, [_VP]),
    "fl_forward_sample": (_I, [_VP, _VP, _VP, _I, _I, _SZ, _VP, C.POINTER(C.c_uint32)]),
    "fl_forward_slots": (_I, [_VP, _VP, _VP, _VP, _I, _I, _VP, _VP]),
    "fl_cache_slot_reset": (_I, [_VP, _I]),
    "fl_cache_slot_len": (_I, [_VP, _I, C.POINTER(_I)]),
    "fl_cache_moe_routing": (_I, [_VP, _I, _VP, _VP]),
    "fl_forward_sample_device": (_I, [_VP, _VP, _VP, _I, _I, _SZ, _VP, C.POINTER(C.c_uint32)]),
    "fl_embed": (_I, [_VP, _VP, _VP, _I, _I, _VP]),
    "fl_embed_timed": (_I, [_VP, _VP, _VP, _I, _I, _VP, _I, C.POINTER(C.c_float)]),
    "fl_comm_unique_id": (_I, [_VP]),
    "fl_comm_init": (_I, [_I, _I, _VP]),
    "fl_comm_ipc_export": (_I, [_VP]),
    "fl_comm_ipc_import": (_I, [_VP, _I, _I]),
    "fl_comm_destroy": (_I, []),
    "fl_prof_begin": (_I, []),
    "fl_prof_end": (_I, [C.c_char_p, _SZ]),
    "fl_launch_count": (_I, [C.POINTER(_U64)]),
}

_lib = None


def load() -> C.CDLL:
    """dlopen the in-tree library and bind every declared symbol.  Raises if the library is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FastllmError(-3, f"{LIB_PATH} is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
                                   "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int):
    if rc != 0:
        raise FastllmError(rc, load().fl_last_error().decode("utf-8", "replace"))


_initialised = None


def init(device: int = 0):
    global _initialised
    if _initialised != device:
        check(load().fl_init(device))
        _initialised = device
