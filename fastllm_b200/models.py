"""Host-side mirror of the reference's trait-based model API over the C ABI.

The reference is Rust and there is no Rust toolchain in this image, so the drop-in host side ships twice:
  * `host/fastllm_host.hpp` -- the C++ mirror (compiled, what INTEGRATION.md's Rust shim is a transliteration of);
  * this module -- the same interface in Python, used by tests/ and bench.py so the parity tests read like the
    reference's own tests (same names, same argument meaning, same offset rules, same error behaviour).

Reference interfaces mirrored (paths under /root/reference/src/models):
  ModelInitializer {initialize_model, initialize_cache, forward}     model_initializer.rs:6-22
  ModelCache {increment_offset, reset, get_offset}                   cache.rs:5-10
  LlamaWithConfig / LlamaCache                                       llama.rs:52-149
  MistralWithConfig / MistralCache                                   mistral.rs:16-236
  QwenWithConfig / QwenCache                                         qwen.rs:12-151
  Model::generate + candle LogitsProcessor (arg-max / temperature)   mod.rs:363-463
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import FastllmError, FlConfig


# --------------------------------------------------------------------------------------------------------------------
# thin RAII handles over the C ABI
# --------------------------------------------------------------------------------------------------------------------
class DeviceModel:
    """fl_model*: device weights (shared between clones)."""

    def __init__(self, cfg, device: int = 0, _handle=None, layers=None):
        """cfg: FlConfig, or FlStackConfig + `layers` (a ctypes array of FlLayerDesc) for a layered model."""
        _lib.init(device)
        self.lib = _lib.load()
        self.cfg = cfg
        self.layers = layers
        self.device = device
        self.vocab = cfg.vocab if isinstance(cfg, _lib.FlStackConfig) else cfg.vocab_size
        if _handle is None:
            h = C.c_void_p()
            if layers is not None:
                _lib.check(self.lib.fl_model_create_layered(C.byref(cfg), layers, C.byref(h)))
            else:
                _lib.check(self.lib.fl_model_create(C.byref(cfg), C.byref(h)))
            self.h = h
        else:
            self.h = _handle

    def put_tensor(self, name: str, arr: np.ndarray):
        if arr.dtype == np.float32:
            dt = _lib.FL_DTYPE_F32
        elif arr.dtype == np.float16:
            dt = _lib.FL_DTYPE_F16
        elif arr.dtype == np.uint16:        # raw bf16 bit patterns
            dt = _lib.FL_DTYPE_BF16
        else:
            raise FastllmError(-1, f"unsupported dtype {arr.dtype} for {name}")
        arr = np.ascontiguousarray(arr)
        shape = (C.c_int64 * arr.ndim)(*arr.shape)
        _lib.check(self.lib.fl_model_put_tensor(self.h, name.encode(), dt, shape, arr.ndim, arr.ctypes.data_as(C.c_void_p)))

    def random_init(self, seed: int = 0, std: float = 0.02):
        _lib.check(self.lib.fl_model_random_init(self.h, seed, std))

    def finalize(self):
        _lib.check(self.lib.fl_model_finalize(self.h))

    def clone(self) -> "DeviceModel":
        h = C.c_void_p()
        _lib.check(self.lib.fl_model_clone(self.h, C.byref(h)))
        return DeviceModel(self.cfg, self.device, _handle=h, layers=self.layers)

    def streamed_bytes(self) -> int:
        n = C.c_uint64()
        _lib.check(self.lib.fl_model_weight_bytes(self.h, C.byref(n)))
        return n.value

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.lib.fl_model_destroy(self.h)
                self.h = None
        except Exception:
            pass


class DeviceCache:
    """fl_cache*: paged KV cache + per-cache stream/workspaces."""

    def __init__(self, model: DeviceModel, max_batch: int, max_seq: int, pool_tokens: int | None = None):
        """pool_tokens (layered models): the cache's pages are a pool of that many tokens shared by the max_batch sequence slots,
        handed out as sequences grow and given back by slot_reset; None = room for max_batch x max_seq tokens."""
        self.model, self.lib = model, model.lib
        self.max_batch, self.max_seq = max_batch, max_seq
        self.vocab = model.vocab
        h = C.c_void_p()
        if pool_tokens is None:
            _lib.check(self.lib.fl_cache_create(model.h, max_batch, max_seq, C.byref(h)))
        else:
            _lib.check(self.lib.fl_cache_create_pooled(model.h, max_batch, max_seq, pool_tokens, C.byref(h)))
        self.h = h

    def forward_ragged(self, slots, token_lists, want=None) -> np.ndarray:
        """One step of a mixed batch (layered models): sequence i lives in slot slots[i] and is fed token_lists[i] (a portion of its
        prompt, or one decoded token) after what the slot already holds.  want: per sequence the places inside its portion whose
        logits are asked for (None = the last token of every portion).  -> f32 [sum of wanted places, vocab], sequence-major."""
        n = len(slots)
        counts = np.asarray([len(t) for t in token_lists], dtype=np.int32)
        if len(token_lists) != n or (counts < 1).any():
            raise FastllmError(-1, "every sequence of a step brings at least one token")
        ids = np.ascontiguousarray(np.concatenate([np.asarray(t, dtype=np.uint32).reshape(-1) for t in token_lists]))
        starts = np.concatenate([[0], np.cumsum(counts)])
        if want is None:
            rows = [int(starts[i + 1]) - 1 for i in range(n)]
        else:
            rows = []
            for i, places in enumerate(want):
                for p in places:
                    if not 0 <= p < counts[i]:
                        raise FastllmError(-1, "a wanted place lies outside its portion")
                    rows.append(int(starts[i]) + int(p))
        rows = np.asarray(rows, dtype=np.int32)
        sl = np.ascontiguousarray(slots, dtype=np.int32)
        out = np.empty((len(rows), self.vocab), dtype=np.float32)
        _lib.check(self.lib.fl_forward_ragged(self.model.h, self.h, sl.ctypes.data_as(C.c_void_p), counts.ctypes.data_as(C.c_void_p), n,
                                              ids.ctypes.data_as(C.c_void_p), rows.ctypes.data_as(C.c_void_p), len(rows),
                                              out.ctypes.data_as(C.c_void_p)))
        return out

    def pool_stats(self):
        """-> (pages of the pool, pages free)"""
        a, b = C.c_int(), C.c_int()
        _lib.check(self.lib.fl_cache_pool_stats(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def reset(self):
        _lib.check(self.lib.fl_cache_reset(self.h))

    def kv_len(self) -> int:
        n = C.c_int()
        _lib.check(self.lib.fl_cache_kv_len(self.h, C.byref(n)))
        return n.value

    def fill_synthetic(self, batch: int, kv_len: int, seed: int = 3):
        _lib.check(self.lib.fl_cache_fill_synthetic(self.h, batch, kv_len, seed))

    def forward(self, ids: np.ndarray, rope_offset: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if ids.ndim != 2:
            raise FastllmError(-1, f"input must be [batch, seq], got shape {ids.shape}")   # input.dims2()? in the reference
        b, t = ids.shape
        out = np.empty((b, self.vocab), dtype=np.float32)
        _lib.check(self.lib.fl_forward(self.model.h, self.h, ids.ctypes.data_as(C.c_void_p), b, t, rope_offset,
                                       out.ctypes.data_as(C.c_void_p)))
        return out

    def forward_greedy(self, ids: np.ndarray, rope_offset: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        b, t = ids.shape
        out = np.empty((b,), dtype=np.uint32)
        _lib.check(self.lib.fl_forward_greedy(self.model.h, self.h, ids.ctypes.data_as(C.c_void_p), b, t, rope_offset,
                                              out.ctypes.data_as(C.c_void_p)))
        return out

    def forward_sample(self, ids: np.ndarray, rope_offset: int, logits_processor: "LogitsProcessor") -> int:
        """fl_forward + LogitsProcessor::sample of row 0 in one call (one V*4-byte read-back, no logits array on this side)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if ids.ndim != 2:
            raise FastllmError(-1, f"input must be [batch, seq], got shape {ids.shape}")
        b, t = ids.shape
        tok = C.c_uint32()
        _lib.check(self.lib.fl_forward_sample(self.model.h, self.h, ids.ctypes.data_as(C.c_void_p), b, t, rope_offset,
                                              logits_processor.h, C.byref(tok)))
        return tok.value

    def forward_sample_device(self, ids: np.ndarray, rope_offset: int, logits_processor: "LogitsProcessor") -> int:
        """The opt-in fast path of forward_sample: soft-max weights, prefix sums and the search run on the device (4 bytes come
        back instead of vocab * 4); the sampler object still owns the generator.  Not bit-identical to the host path by
        construction (block scan instead of a sequential sum): see include/fastllm_b200.h."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if ids.ndim != 2:
            raise FastllmError(-1, f"input must be [batch, seq], got shape {ids.shape}")
        b, t = ids.shape
        tok = C.c_uint32()
        _lib.check(self.lib.fl_forward_sample_device(self.model.h, self.h, ids.ctypes.data_as(C.c_void_p), b, t, rope_offset,
                                                     logits_processor.h, C.byref(tok)))
        return tok.value

    def forward_slots(self, slots, ids: np.ndarray, rope_offsets) -> np.ndarray:
        """Ragged forward (continuous batching): row i of ids [n, t] is fed to the sequence in cache slot slots[i] at RoPE
        position rope_offsets[i]; the slots keep their own lengths.  -> f32 [n, vocab]."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if ids.ndim != 2:
            raise FastllmError(-1, f"input must be [batch, seq], got shape {ids.shape}")
        n, t = ids.shape
        sl = np.ascontiguousarray(slots, dtype=np.int32).reshape(-1)
        ro = np.ascontiguousarray(rope_offsets, dtype=np.uint64).reshape(-1)
        if sl.size != n or ro.size != n:
            raise FastllmError(-1, "slots / rope_offsets must have one entry per row of ids")
        out = np.empty((n, self.vocab), dtype=np.float32)
        _lib.check(self.lib.fl_forward_slots(self.model.h, self.h, sl.ctypes.data_as(C.c_void_p), ids.ctypes.data_as(C.c_void_p), n, t,
                                             ro.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)))
        return out

    def slot_reset(self, slot: int):
        _lib.check(self.lib.fl_cache_slot_reset(self.h, slot))

    def slot_len(self, slot: int) -> int:
        n = C.c_int()
        _lib.check(self.lib.fl_cache_slot_len(self.h, slot, C.byref(n)))
        return n.value

    def moe_routing(self, rows: int):
        """Router decisions of the last forward (Mixtral): experts [layers, rows, top_k] int32 in pick order, margins [layers, rows] f32."""
        cfg = self.model.cfg
        ex = np.empty((cfg.num_hidden_layers, rows, cfg.num_experts_per_tok), dtype=np.int32)
        mg = np.empty((cfg.num_hidden_layers, rows), dtype=np.float32)
        _lib.check(self.lib.fl_cache_moe_routing(self.h, rows, ex.ctypes.data_as(C.c_void_p), mg.ctypes.data_as(C.c_void_p)))
        return ex, mg

    def decode_greedy_loop(self, first_ids: np.ndarray, rope_offset: int, steps: int):
        first = np.ascontiguousarray(first_ids, dtype=np.uint32).reshape(-1)
        b = first.shape[0]
        out = np.empty((steps, b), dtype=np.uint32)
        ms = C.c_float()
        _lib.check(self.lib.fl_decode_greedy_loop(self.model.h, self.h, first.ctypes.data_as(C.c_void_p), b, rope_offset,
                                                  steps, out.ctypes.data_as(C.c_void_p), C.byref(ms)))
        return out, ms.value

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.lib.fl_cache_destroy(self.h)
                self.h = None
        except Exception:
            pass


def prof_begin():
    _lib.check(_lib.load().fl_prof_begin())


def prof_end() -> list:
    buf = C.create_string_buffer(1 << 16)
    _lib.check(_lib.load().fl_prof_end(buf, len(buf)))
    return json.loads(buf.value.decode())


def launch_count() -> int:
    n = C.c_uint64()
    _lib.check(_lib.load().fl_launch_count(C.byref(n)))
    return n.value


# --------------------------------------------------------------------------------------------------------------------
# configs (what the adapters deserialize from config.json)
# --------------------------------------------------------------------------------------------------------------------
@dataclass
class ConfigFile:
    """llama.rs:17-29 / mistral.rs:78-91 / models/config.rs:5-18 (BaseModelConfig)."""
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int | None = None
    rms_norm_eps: float = 1e-5
    rope_theta: float | None = None
    max_position_embeddings: int | None = None
    sliding_window: int | None = None
    torch_dtype: str | None = None     # never consulted by the reference (huggingface.rs:132)
    tp_rank: int = 0                   # tensor parallelism (no reference counterpart): rank / size of this process
    tp_size: int = 1                   # (for Mixtral the same two fields mean expert-parallel rank / size)
    num_local_experts: int = 0         # Mixtral
    num_experts_per_tok: int = 2
    ep_dp_attention: bool = False      # Mixtral expert parallelism: sequences data-parallel, tokens all-to-all to the experts


def _fl_config(arch: str, cf: ConfigFile, default_max_pos: int, sliding_window: int, qkv_bias: bool) -> FlConfig:
    c = FlConfig()
    c.arch = _lib.FL_ARCH[arch]
    c.hidden_size, c.intermediate_size, c.vocab_size = cf.hidden_size, cf.intermediate_size, cf.vocab_size
    c.num_hidden_layers, c.num_attention_heads = cf.num_hidden_layers, cf.num_attention_heads
    c.num_key_value_heads = cf.num_key_value_heads or cf.num_attention_heads
    c.max_position_embeddings = cf.max_position_embeddings or default_max_pos
    c.sliding_window = sliding_window
    c.qkv_bias = 1 if qkv_bias else 0
    c.norm_eps = cf.rms_norm_eps
    c.rope_theta = float(cf.rope_theta if cf.rope_theta is not None else 10000.0)
    c.tp_rank, c.tp_size = cf.tp_rank, cf.tp_size
    c.num_local_experts, c.num_experts_per_tok = cf.num_local_experts, cf.num_experts_per_tok
    c.ep_dp_attention = 1 if cf.ep_dp_attention else 0
    return c


# --------------------------------------------------------------------------------------------------------------------
# ModelCache implementations
# --------------------------------------------------------------------------------------------------------------------
class _OffsetCache:
    """ModelCache (cache.rs:5-10): increment_offset / reset / get_offset."""

    def __init__(self):
        self.seqlen_offset = 0

    def increment_offset(self):
        self.seqlen_offset += 1

    def reset(self):
        self.seqlen_offset = 0

    def get_offset(self) -> int:
        return self.seqlen_offset


class LlamaCache(_OffsetCache):
    """llama.rs:61-92.  In the reference this owns candle's KV `Cache`; here it owns the device KV cache, created lazily
    on the first forward because initialize_cache(device, dtype) gets no model argument."""

    def __init__(self):
        super().__init__()
        self.inner: DeviceCache | None = None


class MistralCache(_OffsetCache):
    """mistral.rs:16-47: only the offset; the KV lives inside the model object."""


class QwenCache(_OffsetCache):
    """qwen.rs:58-87."""


# --------------------------------------------------------------------------------------------------------------------
# ModelInitializer implementations
# --------------------------------------------------------------------------------------------------------------------
class _CausalBase:
    arch = ""
    family = ""
    architectures: tuple = ()
    KV_CAPACITY = 4096        # tokens of KV a cache can hold (the reference grows by `cat`; we preallocate pages)
    MAX_BATCH = 1

    def __init__(self, dev: DeviceModel, cfg: FlConfig):
        self.dev, self.cfg = dev, cfg

    @classmethod
    def _to_fl_config(cls, config: ConfigFile) -> FlConfig:
        raise NotImplementedError

    @classmethod
    def initialize_model(cls, config: ConfigFile, tensors: dict | None, dtype="bf16", device: int = 0, *, random_seed=None,
                         std: float = 0.02):
        """ModelInitializer::initialize_model(&Config, HashMap<String,Tensor>, DType, &Device) -> (Self, Cache).
        `tensors` maps HF names to numpy arrays (f32 / f16 / uint16 bf16 bits); they are rounded to bf16 as
        VarBuilder::from_tensors(.., BF16, ..) would (main.rs:120).  tensors=None + random_seed = synthetic weights."""
        cfg = cls._to_fl_config(config)
        dev = DeviceModel(cfg, device)
        if tensors is None:
            dev.random_init(0 if random_seed is None else random_seed, std)
        else:
            # a dict, or any iterable of (name, array) -- e.g. safetensors_io.iter_tensors(dir), which hands over views of the
            # memory-mapped checkpoint one tensor at a time (huggingface.rs:81-130 without the whole-file reads)
            for name, arr in (tensors.items() if hasattr(tensors, "items") else tensors):
                dev.put_tensor(name, np.asarray(arr))
        dev.finalize()
        self = cls(dev, cfg)
        return self, cls.initialize_cache(device, dtype)

    @classmethod
    def get_family(cls) -> str:
        return cls.family

    @classmethod
    def supports_architecture(cls, architecture: str) -> bool:
        return architecture in cls.architectures

    def _capacity(self) -> int:
        return min(self.KV_CAPACITY, self.cfg.max_position_embeddings)


class LlamaWithConfig(_CausalBase):
    """llama.rs:52-160."""
    arch, family, architectures = "llama", "Llama", ("LlamaForCausalLM",)

    @classmethod
    def _to_fl_config(cls, cf: ConfigFile) -> FlConfig:
        # llama.rs:31-50: rope_theta default 1e4, max_position_embeddings default 4096, no sliding window, no bias
        return _fl_config("llama", cf, 4096, 0, False)

    @staticmethod
    def initialize_cache(device=0, dtype="bf16") -> LlamaCache:
        return LlamaCache()

    def forward(self, input: np.ndarray, pos: int, cache: LlamaCache) -> np.ndarray:
        """llama.rs:147-149: model.forward(input, pos, &mut cache.inner) -> f32 [b, V]."""
        ids = np.asarray(input)
        if cache.inner is None:
            cache.inner = DeviceCache(self.dev, max(self.MAX_BATCH, ids.shape[0] if ids.ndim == 2 else 1), self._capacity())
        return cache.inner.forward(ids, pos)

    def clone(self) -> "LlamaWithConfig":
        return LlamaWithConfig(self.dev.clone(), self.cfg)


class MistralWithConfig(_CausalBase):
    """mistral.rs:49-248.  The KV cache lives in the model object (one per clone), as in candle's mistral::Model."""
    arch, family, architectures = "mistral", "Mistral", ("MistralForCausalLM",)
    cache_cls = MistralCache

    def __init__(self, dev: DeviceModel, cfg: FlConfig):
        super().__init__(dev, cfg)
        self._kv: DeviceCache | None = None

    @classmethod
    def _to_fl_config(cls, cf: ConfigFile) -> FlConfig:
        # mistral.rs:93-154: asserts on head dims / GQA (raised as FastllmError by fl_model_create),
        # sliding_window = Some(cfg.unwrap_or(4096)), max_position_embeddings default 32768
        return _fl_config("mistral", cf, 32768, cf.sliding_window if cf.sliding_window is not None else 4096, False)

    @classmethod
    def initialize_cache(cls, device=0, dtype="bf16"):
        return cls.cache_cls()

    def clear_kv_cache(self):
        if self._kv is not None:
            self._kv.reset()

    def forward(self, input: np.ndarray, _pos: int, cache) -> np.ndarray:
        """mistral.rs:206-236 / qwen.rs:129-145: `_pos` ignored; KV cleared when the offset is 0; RoPE offset = the
        cache's seqlen_offset, which then grows by ONE per call (not by seq_len).  Returns [b, 1, V]."""
        ids = np.asarray(input)
        if ids.ndim != 2:
            raise FastllmError(-1, f"input must be [batch, seq], got shape {ids.shape}")
        if self._kv is None or (cache.get_offset() == 0 and self._kv.max_batch < ids.shape[0]):
            self._kv = DeviceCache(self.dev, max(self.MAX_BATCH, ids.shape[0]), self._capacity())   # a wider batch starts a new KV
        if cache.get_offset() == 0:
            self.clear_kv_cache()
        out = self._kv.forward(ids, cache.get_offset())
        cache.increment_offset()
        return out[:, None, :]

    def clone(self):
        return type(self)(self.dev.clone(), self.cfg)


class QwenWithConfig(MistralWithConfig):
    """qwen.rs:12-186 (ModelForward::forward_pass + clear_cache; q/k/v bias)."""
    arch, family = "qwen2", "Qwen"
    architectures = ("Qwen2ForCausalLM", "Qwen2_5_VLForConditionalGeneration")
    cache_cls = QwenCache

    @classmethod
    def _to_fl_config(cls, cf: ConfigFile) -> FlConfig:
        # qwen.rs:30-56: sliding_window.unwrap_or(4096), max_position_embeddings default 32768, rope default 1e4
        return _fl_config("qwen2", cf, 32768, cf.sliding_window if cf.sliding_window is not None else 4096, True)

    def forward_pass(self, input, cache):
        return self.forward(input, 0, cache)

    def clear_cache(self):
        self.clear_kv_cache()


class MixtralWithConfig(MistralWithConfig):
    """MixtralForCausalLM.  The reference does NOT wire this architecture (model_registry.rs:169-182 has no matching key,
    mistral.rs:244-246 accepts only MistralForCausalLM); the adapter follows the Mistral one (same offset rule) over
    candle-transformers' mixtral model: attention as Mistral, MLP replaced by the top-k sparse-MoE block."""
    arch, family, architectures = "mixtral", "Mixtral", ("MixtralForCausalLM",)

    @classmethod
    def _to_fl_config(cls, cf: ConfigFile) -> FlConfig:
        return _fl_config("mixtral", cf, 32768, cf.sliding_window if cf.sliding_window is not None else 4096, False)


class NifunexCache(_OffsetCache):
    """Cache handle of the layered decoders: owns the device cache (latent pages + recurrent-state slots), created on first use."""

    def __init__(self):
        super().__init__()
        self.inner: DeviceCache | None = None


def nifunex_layer_descs(config: dict, decay_ranks: dict):
    """config.json of the layered decoder -> ctypes array of FlLayerDesc.  decay_ranks: layer index -> rows of that layer's decay
    bottleneck (the one size the file does not spell out; it is the first dimension of 'l<i>.mix.a1')."""
    layers = config["layers"]
    arr = (_lib.FlLayerDesc * len(layers))()
    for i, l in enumerate(layers):
        d, m = arr[i], l["mixer"]
        if l["type"] not in ("gla", "latent_attention"):
            raise FastllmError(-1, f"layer {i}: unknown mixer type {l['type']!r}")
        d.mixer = _lib.FL_MIXER[l["type"]]
        d.heads, d.dim, d.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        d.kv_from = -1
        if l["type"] == "gla":
            d.tau = float(m["tau"])
            if i not in decay_ranks:
                raise FastllmError(-1, f"layer {i}: the decay bottleneck's size is unknown (no 'l{i}.mix.a1' tensor and no decay_rank)")
            d.decay_rank = int(decay_ranks[i])
        else:
            d.rot_dim, d.kv_rank = int(m["rot_dim"]), int(m["kv_rank"])
            d.kv_from = int(m["kv_from"]) if m.get("kv_from") is not None else -1
            d.window = int((m.get("mask") or {}).get("size") or 0)
            d.scale = float(m["scale"])
            _rotary_desc(d, m.get("rot") or {}, d.rot_dim)
        _ffn_desc(d, i, l.get("mlp"))
    return arr


def _ffn_desc(d, i: int, mlp, act: str = "swish_clamp", bias: bool = False):
    """fills the feed-forward fields of a FlLayerDesc from a layer's 'mlp' entry (None = the layer has none)"""
    d.ffn_act, d.ffn_bias = _lib.FL_ACT[act], 1 if bias else 0
    if not mlp:
        d.ffn = _lib.FL_FFN["none"]
    elif mlp["kind"] == "dense":
        d.ffn, d.ff, d.limit = _lib.FL_FFN["dense"], int(mlp["ff"]), float(mlp.get("limit", 0.0))
    elif mlp["kind"] == "moe":
        d.ffn, d.ff, d.limit = _lib.FL_FFN["moe"], int(mlp["expert"]["ff"]), float(mlp["expert"]["limit"])
        d.experts, d.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        if mlp.get("shared"):
            d.shared_ff, d.shared_limit = int(mlp["shared"]["ff"]), float(mlp["shared"]["limit"])
    else:
        raise FastllmError(-1, f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")


def _rotary_desc(d, rot: dict, default_dims: int):
    """fills the rotary fields (leading rotated channels, base, optional YaRN scaling) from a mixer's 'rot' entry"""
    d.rot_dims = int(rot.get("dims", default_dims))
    d.rot_base = float(rot.get("base", 10000.0))
    sc = rot.get("scaling")
    if sc:
        d.yarn_factor, d.yarn_original = float(sc["factor"]), float(sc["original"])
        d.yarn_fast, d.yarn_slow = float(sc["fast"]), float(sc["slow"])


class _LayeredBase(_CausalBase):
    """Adapters of the layered decoders: `config` is the parsed config.json (a dict: vocab, width, norm.eps and one entry per
    layer).  A subclass names its architecture, its norm conventions and how a layer entry becomes a FlLayerDesc.  Positions are
    the caller's, as for Llama; the device cache hands out pages on demand and keeps a recurrent-state slot per sequence."""
    position_per_call = False
    MAX_BATCH = 1
    POOL_TOKENS = None          # None: room for MAX_BATCH x capacity tokens
    norm_plain = False          # layer norms and the final norm scale by w instead of 1 + w
    no_pre_norm = False         # sublayers read the residual stream itself; only their outputs are normed
    no_post_norm = False        # a sublayer's result joins the residual stream as it is

    @classmethod
    def stack_options(cls, config: dict, sc) -> None:
        """fills the stack-wide options of a FlStackConfig that the design reads from config.json (none by default)"""

    @classmethod
    def config_tensors(cls, config: dict):
        """(name, f32 array) pairs the design states in config.json rather than in the checkpoint (per-head constants and the like);
        they reach the device as tensors of those names, bit for bit"""
        return ()

    def __init__(self, dev: DeviceModel, cfg, config: dict):
        super().__init__(dev, cfg)
        self.config = config

    @classmethod
    def layer_descs(cls, config: dict, tensor_shapes: dict, **hints):
        """config.json (+ the shapes of the checkpoint's tensors, for sizes the file does not spell out) -> ctypes array of FlLayerDesc"""
        raise NotImplementedError

    @classmethod
    def initialize_model(cls, config: dict, tensors, dtype="bf16", device: int = 0, *, random_seed=None, std: float = 0.02, **hints):
        """tensors: dict or iterable of (name, array) (f32 / f16 / uint16 bf16 bits), or None for synthetic weights.  dtype "bf16":
        the serving precision; "f32": every product and the cache in true 32-bit."""
        if dtype not in ("bf16", "bfloat16", "f32", "float32"):
            raise FastllmError(-1, f"unsupported dtype {dtype!r}")
        items, shapes = None, {}
        if tensors is not None:
            items = list(tensors.items() if hasattr(tensors, "items") else tensors)
            shapes = {name: tuple(np.asarray(arr).shape) for name, arr in items}
        sc = _lib.FlStackConfig()
        sc.arch = _lib.FL_ARCH[cls.arch]
        sc.vocab, sc.width, sc.n_layers = int(config["vocab"]), int(config["width"]), len(config["layers"])
        sc.norm_eps = float(config["norm"]["eps"])
        sc.compute_dtype = _lib.FL_DTYPE_F32 if dtype in ("f32", "float32") else _lib.FL_DTYPE_BF16
        sc.norm_plain, sc.no_pre_norm, sc.no_post_norm = int(cls.norm_plain), int(cls.no_pre_norm), int(cls.no_post_norm)
        cls.stack_options(config, sc)
        dev = DeviceModel(sc, device, layers=cls.layer_descs(config, shapes, **hints))
        if items is None:
            dev.random_init(0 if random_seed is None else random_seed, std)
        else:
            for name, arr in items:
                a = np.asarray(arr)
                if a.dtype.kind in "iu" and a.dtype != np.uint16:
                    continue            # integer tables: these designs read none
                dev.put_tensor(name, a)
        for name, arr in cls.config_tensors(config):
            dev.put_tensor(name, np.ascontiguousarray(arr, dtype=np.float32))
        dev.finalize()
        self = cls(dev, sc, config)
        return self, cls.initialize_cache(device, dtype)

    @staticmethod
    def initialize_cache(device=0, dtype="bf16") -> NifunexCache:
        return NifunexCache()

    def _capacity(self) -> int:
        return self.KV_CAPACITY

    def new_device_cache(self, max_batch: int | None = None, max_seq: int | None = None, pool_tokens: int | None = None) -> DeviceCache:
        return DeviceCache(self.dev, max_batch or self.MAX_BATCH, max_seq or self._capacity(), pool_tokens if pool_tokens is not None else self.POOL_TOKENS)

    def forward(self, input: np.ndarray, pos: int, cache: NifunexCache) -> np.ndarray:
        """[b, t] token ids at positions pos.. -> f32 [b, V] logits of the last position (pos must equal what the cache holds)."""
        ids = np.asarray(input)
        if ids.ndim != 2:
            raise FastllmError(-1, f"input must be [batch, seq], got shape {ids.shape}")
        if cache.inner is None:
            cache.inner = self.new_device_cache(max(self.MAX_BATCH, ids.shape[0]))
        return cache.inner.forward(ids, pos)

    def clone(self):
        return type(self)(self.dev.clone(), self.cfg, self.config)


class NifunexWithConfig(_LayeredBase):
    """The Nifunex decoder (no reference path): gated-linear-attention and windowed latent-attention layers, dense / MoE
    feed-forward, norms with a zero-centred weight before and after every sublayer."""
    arch, family, architectures = "nifunex", "Nifunex", ("Nifunex",)

    @classmethod
    def layer_descs(cls, config: dict, tensor_shapes: dict, decay_rank=None):
        """the decay bottleneck's rows are the one size config.json does not spell out: the first dimension of 'l<i>.mix.a1', or
        decay_rank for synthetic weights"""
        ranks = {}
        for name, shp in tensor_shapes.items():
            if name.endswith(".mix.a1") and name[0] == "l":
                ranks[int(name[1:name.index(".")])] = int(shp[0])
        if not tensor_shapes:
            ranks = {i: int(decay_rank or 16) for i, l in enumerate(config["layers"]) if l["type"] == "gla"}
        return nifunex_layer_descs(config, ranks)


def rofetar_layer_descs(config: dict):
    """config.json of the Rofetar decoder -> ctypes array of FlLayerDesc (every size and constant comes from the file)."""
    layers = config["layers"]
    arr = (_lib.FlLayerDesc * len(layers))()
    for i, l in enumerate(layers):
        d, m, kind = arr[i], l["mixer"], l["type"]
        if kind not in ("attention", "mamba2", "delta"):
            raise FastllmError(-1, f"layer {i}: unknown mixer type {kind!r}")
        d.mixer = _lib.FL_MIXER[kind]
        d.heads, d.vdim = int(m["heads"]), int(m["vdim"])
        d.kv_from = -1
        if kind == "attention":
            d.dim, d.kv_heads = int(m["dim"]), int(m.get("kv_heads") or m["heads"])
            d.kv_from = int(m["kv_from"]) if m.get("kv_from") is not None else -1
            d.scale = float(m["scale"])
            d.softcap = float(m.get("softcap") or 0.0)
            d.sink, d.rot_halves = 1, 1
            _rotary_desc(d, m.get("rot") or {"dims": 0}, 0)
        elif kind == "mamba2":
            d.state, d.groups, d.conv = int(m["state"]), int(m.get("groups") or 1), int(m["conv"])
            d.norm_groups = int(m.get("norm_groups") or 1)
        else:
            d.dim, d.kv_heads, d.conv = int(m["dim"]), int(m.get("kv_heads") or m["heads"]), int(m["conv"])
        _ffn_desc(d, i, l.get("mlp"), act="gelu_tanh", bias=True)
        if d.ffn == _lib.FL_FFN["moe"]:
            raise FastllmError(-1, f"layer {i}: this design has dense feed-forwards only")
    return arr


class RofetarWithConfig(_LayeredBase):
    """The Rofetar decoder (no reference path): grouped-query attention with per-head q/k norms, a score cap and a softmax sink
    (optionally on another layer's keys and values), Mamba-2 and gated-delta-rule layers, a biased tanh-gelu feed-forward; a
    sublayer reads the residual stream as it is and only its output is normed (plain weight)."""
    arch, family, architectures = "rofetar", "Rofetar", ("Rofetar",)
    norm_plain, no_pre_norm = True, True

    @classmethod
    def layer_descs(cls, config: dict, tensor_shapes: dict):
        return rofetar_layer_descs(config)


def _attention_desc(d, m: dict):
    """fills the fields of a plain grouped-query attention mixer (no q/k norm, no rotation unless 'rot' says so, optional window)"""
    d.mixer = _lib.FL_MIXER["attention"]
    d.heads, d.dim, d.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    d.kv_heads, d.kv_from = int(m.get("kv_heads") or m["heads"]), -1
    d.scale = float(m["scale"])
    d.window = int((m.get("mask") or {}).get("size") or 0)
    d.no_qk_norm, d.rot_halves = 1, 1
    _rotary_desc(d, m.get("rot") or {"dims": 0}, 0)


def _delta_desc(d, m: dict):
    """fills the fields of a gated-delta-rule mixer"""
    d.mixer = _lib.FL_MIXER["delta"]
    d.heads, d.dim, d.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    d.kv_heads, d.conv, d.kv_from = int(m.get("kv_heads") or m["heads"]), int(m["conv"]), -1


def tozarax_layer_descs(config: dict):
    """config.json of the Tozarax decoder -> ctypes array of FlLayerDesc: two descriptors per layer (the attention mixer with the
    layer's feed-forward, then the delta-rule mixer that runs beside it).  Every size and constant comes from the file."""
    layers = config["layers"]
    arr = (_lib.FlLayerDesc * (2 * len(layers)))()
    for i, l in enumerate(layers):
        if l["type"] != "parallel":
            raise FastllmError(-1, f"layer {i}: unknown mixer type {l['type']!r}")
        a, b = arr[2 * i], arr[2 * i + 1]
        _attention_desc(a, l["mixer"]["left"])
        a.beside = 1
        _delta_desc(b, l["mixer"]["right"])
        mlp = l.get("mlp")
        if not mlp:
            a.ffn = _lib.FL_FFN["none"]
            continue
        if mlp["kind"] != "moe":
            raise FastllmError(-1, f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        r = mlp["router"]
        a.ffn, a.ffn_act, a.ff = _lib.FL_FFN["moe"], _lib.FL_ACT["relu2"], int(mlp["expert"]["ff"])
        a.experts, a.top = int(r["experts"]), int(r["top"])
        a.router = _lib.FL_ROUTER["sigmoid_groups"]
        g = r.get("groups") or {}
        a.route_groups = int(g.get("count") or 1)
        a.route_keep = int(g.get("keep") or a.route_groups)
    return arr


class TozaraxWithConfig(_LayeredBase):
    """The Tozarax decoder (no reference path): learned positions; every layer runs a windowed softmax attention without rotation
    beside a gated delta rule (each output normed, the two averaged) and a sigmoid-routed mixture of squared-relu experts with
    group-limited choice; sublayers are pre-normed, read their input through a short causal convolution, scale their contribution
    by a learned gate, and every layer hands on a learned average of all layers' outputs so far."""
    arch, family, architectures = "tozarax", "Tozarax", ("Tozarax",)
    no_post_norm = True

    @classmethod
    def stack_options(cls, config: dict, sc) -> None:
        sc.max_positions = int(config.get("max_positions") or 0)
        sc.canon_taps = int((config.get("canon") or {}).get("taps") or 0)
        sc.gated_residual, sc.depth_avg = 1, 1

    @classmethod
    def layer_descs(cls, config: dict, tensor_shapes: dict):
        return tozarax_layer_descs(config)

    def _capacity(self) -> int:
        return min(self.KV_CAPACITY, int(self.config.get("max_positions") or self.KV_CAPACITY))


def _rotary_bands_desc(d, rot: dict):
    """rotary fields with Llama-3.1 style frequency scaling: 'scaling' = {factor, low, high, original}"""
    d.rot_dims = int(rot.get("dims") or 0)
    d.rot_base = float(rot.get("base", 10000.0))
    sc = rot.get("scaling")
    if sc:
        d.rot_scaling = _lib.FL_ROT_SCALE["bands"]
        d.yarn_factor, d.yarn_original = float(sc["factor"]), float(sc["original"])
        d.yarn_fast, d.yarn_slow = float(sc["high"]), float(sc["low"])


def _medulorn_softmax_desc(d, m: dict, windowed: bool):
    """the two softmax attentions of the Medulorn decoder: chunk-masked with biased projections, per-head q/k norm and a sink of
    score zero; or windowed with kept first tokens, q/k norm over the whole projection and a learned sink per head"""
    d.mixer = _lib.FL_MIXER["attention"]
    d.heads, d.dim, d.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    d.kv_heads, d.kv_from = int(m.get("kv_heads") or m["heads"]), -1
    d.scale, d.rot_halves = float(m["scale"]), 1
    mask = m.get("mask") or {}
    if windowed:
        d.window, d.keep_first = int(mask.get("size") or 0), int(mask.get("keep_first") or 0)
        d.qk_norm_whole, d.sink = 1, 2
    else:
        d.mask_chunk = int(mask.get("size") or 0)
        d.qkv_bias, d.sink = 1, 1
    _rotary_bands_desc(d, m.get("rot") or {})


def medulorn_layer_descs(config: dict):
    """config.json of the Medulorn decoder -> ctypes array of FlLayerDesc: one descriptor for an 'attention' layer, two for a
    'parallel' one (the windowed attention with the layer's feed-forward, then the lightning attention beside it).  Every size
    and constant comes from the file."""
    layers = config["layers"]
    for i, l in enumerate(layers):
        if l["type"] not in ("attention", "parallel"):
            raise FastllmError(-1, f"layer {i}: unknown mixer type {l['type']!r}")
    arr = (_lib.FlLayerDesc * sum(2 if l["type"] == "parallel" else 1 for l in layers))()
    k = 0
    for i, l in enumerate(layers):
        a, m = arr[k], l["mixer"]
        k += 1
        if l["type"] == "attention":
            _medulorn_softmax_desc(a, m, windowed=False)
        else:
            _medulorn_softmax_desc(a, m["left"], windowed=True)
            a.beside, a.pair_sum, a.out_scale = 1, 1, float(m["left_scale"])
            b, r = arr[k], m["right"]
            k += 1
            b.mixer, b.kv_from = _lib.FL_MIXER["lightning"], -1
            b.heads, b.dim, b.vdim = int(r["heads"]), int(r["dim"]), int(r["vdim"])
            b.out_scale = float(m["right_scale"])
            if len(r["decay"]) != b.heads:
                raise FastllmError(-1, f"layer {i}: one decay per head is needed")
        mlp = l.get("mlp")
        _ffn_desc(a, i, mlp, act="relu" if (mlp and mlp["kind"] == "dense") else "swish_clamp")
        if a.ffn == _lib.FL_FFN["moe"]:
            a.router_bias, a.shared_plain = 1, 1
    return arr


class MedulornWithConfig(_LayeredBase):
    """The Medulorn decoder (no reference path): x <- norm(alpha x + sublayer(x)) with one number as every norm's weight; mixers read
    x through a token shift; 'attention' layers (chunk mask, biased projections, sink of score zero) and 'parallel' layers (windowed
    attention with kept first tokens and a learned sink, beside lightning attention, summed with fixed shares); a relu-gated dense
    feed-forward or clamped-swish experts with a biased router and an ungated shared expert; scaled embedding, capped logits."""
    arch, family, architectures = "medulorn", "Medulorn", ("Medulorn",)
    norm_plain, no_pre_norm = True, True

    @classmethod
    def stack_options(cls, config: dict, sc) -> None:
        sc.post_sum_norm, sc.residual_alpha = 1, float(config.get("postln_alpha", 1.0))
        sc.norm_scalar, sc.token_shift = 1, 1
        sc.embed_scale = float((config.get("embedding") or {}).get("scale") or 0.0)
        sc.logit_softcap = float(config.get("logit_softcap") or 0.0)

    @classmethod
    def layer_descs(cls, config: dict, tensor_shapes: dict):
        return medulorn_layer_descs(config)

    @classmethod
    def config_tensors(cls, config: dict):
        for i, l in enumerate(config["layers"]):
            if l["type"] == "parallel":
                yield f"l{i}.mix.right.decay", np.asarray(l["mixer"]["right"]["decay"], dtype=np.float32)


# every adapter, in the order the registry tries them (model_registry.rs:169-182 keeps the same kind of list)
def registered_models():
    return (LlamaWithConfig, MistralWithConfig, QwenWithConfig, MixtralWithConfig, NifunexWithConfig, RofetarWithConfig, TozaraxWithConfig,
            MedulornWithConfig)


def model_class_for(config: dict):
    """The adapter whose supports_architecture accepts the config.json's `architectures` list (HF) or `architecture` name."""
    names = list(config.get("architectures") or [])
    if config.get("architecture"):
        names.append(config["architecture"])
    for cls in registered_models():
        if any(cls.supports_architecture(n) for n in names):
            return cls
    raise FastllmError(-5, f"no registered model supports {names}")


def load_model(model_dir: str, dtype: str = "bf16", device: int = 0):
    """config.json + safetensors of a folder -> (adapter instance, cache handle), the class chosen by the registry."""
    import os
    from . import safetensors_io
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    cls = model_class_for(config)
    if issubclass(cls, _LayeredBase):
        return cls.initialize_model(config, safetensors_io.iter_tensors(model_dir, copy=True), dtype, device)
    cf = ConfigFile(config["hidden_size"], config["intermediate_size"], config["vocab_size"], config["num_hidden_layers"],
                    config["num_attention_heads"], config.get("num_key_value_heads"), config.get("rms_norm_eps", 1e-5),
                    config.get("rope_theta"), config.get("max_position_embeddings"), config.get("sliding_window"),
                    num_local_experts=config.get("num_local_experts", 0), num_experts_per_tok=config.get("num_experts_per_tok", 2))
    return cls.initialize_model(cf, safetensors_io.iter_tensors(model_dir), dtype, device)


class LogitsProcessor:
    """candle's LogitsProcessor as the reference builds it: LogitsProcessor::new(Default::default(), Some(temperature as f64),
    None) (mod.rs:157-158, 373-374).  Temperature < 1e-7 => arg-max (IEEE total order, LAST index among equal maxima);
    otherwise soft-max + WeightedIndex over StdRng::seed_from_u64(seed).  The arithmetic is the library's (fl_sampler_*,
    csrc/sampler.hpp): host code, because the reference samples on the host from the logits every forward returns."""

    def __init__(self, seed: int = 0, temperature: float | None = None):
        self.lib = _lib.load()
        h = C.c_void_p()
        _lib.check(self.lib.fl_sampler_create(seed, -1.0 if temperature is None else float(temperature), C.byref(h)))
        self.h = h

    def sample(self, logits: np.ndarray) -> int:
        v = np.ascontiguousarray(logits, dtype=np.float32).reshape(-1)       # logits.to_dtype(F32)
        tok = C.c_uint32()
        _lib.check(self.lib.fl_sampler_sample(self.h, v.ctypes.data_as(C.c_void_p), v.size, C.byref(tok)))
        return tok.value

    def next_u32(self) -> int:
        w = C.c_uint32()
        _lib.check(self.lib.fl_sampler_next_u32(self.h, C.byref(w)))
        return w.value

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.lib.fl_sampler_destroy(self.h)
                self.h = None
        except Exception:
            pass


def sample_argmax(logits: np.ndarray) -> int:
    """LogitsProcessor::sample with temperature None/<1e-7: arg-max, LAST index among equal maxima (mod.rs:425-428)."""
    global _greedy
    if _greedy is None:
        _greedy = LogitsProcessor(0, None)      # arg-max never touches the generator: one shared instance
    return _greedy.sample(logits)


_greedy = None


def sample_argmax_rows(logits: np.ndarray) -> np.ndarray:
    """sample_argmax for every row of [b, V] logits (a batch of greedy requests) in one library call -> u32 [b]."""
    v = np.ascontiguousarray(logits, dtype=np.float32)
    v = v.reshape(v.shape[0], -1)
    out = np.empty((v.shape[0],), dtype=np.uint32)
    _lib.check(_lib.load().fl_argmax_rows(v.ctypes.data_as(C.c_void_p), v.shape[0], v.shape[1], out.ctypes.data_as(C.c_void_p)))
    return out


class Model:
    """Model<M> (mod.rs:342-464) without the tokenizer: prompts are already token ids."""

    def __init__(self, model, cache, eos_token_id: int | None = 2):
        self.model, self.cache, self.eos_token_id = model, cache, eos_token_id

    def generate(self, prompt_ids, max_tokens: int, temperature: float = 0.0, return_logits: bool = False):
        self.cache = self.model.initialize_cache()                       # mod.rs:370
        # mod.rs:373-374: seed Default::default() = 0, `temperature as f64` of the API's f32 (chat.rs:24-25 defaults it to 0.0)
        logits_processor = LogitsProcessor(0, float(np.float32(temperature)))
        ids = np.asarray(prompt_ids, dtype=np.uint32).reshape(1, -1)    # mod.rs:386-394
        pos = 0
        logits = self.model.forward(ids, pos, self.cache)               # mod.rs:402-405
        pos += ids.shape[1]
        out, trace = [], []
        for _ in range(max_tokens):                                      # mod.rs:411-453
            last = np.asarray(logits)[0].reshape(-1)                     # logits.get(0)?.flatten_all()?
            if return_logits:
                trace.append(last.copy())
            tok = logits_processor.sample(last)                          # mod.rs:425-428
            if self.eos_token_id is not None and tok == self.eos_token_id:
                break                                                    # EOS: break before emitting (mod.rs:431-436)
            out.append(tok)
            logits = self.model.forward(np.array([[tok]], dtype=np.uint32), pos, self.cache)
            pos += 1
        return (out, trace) if return_logits else out

    def generate_batch(self, prompts, max_tokens: int, temperature: float = 0.0, max_batch: int = 64):
        """Request batching at the API boundary (the reference serialises requests at batch 1 under a
        mutex, chat.rs:206-208).  Exact by construction: only prompts of EQUAL token length share a batch, so the sequences of
        a group advance in lock-step through one [b, t] forward per step (no padding, one KV length), every sequence has its
        own LogitsProcessor seeded 0 like every request of the reference, and a sequence that hit EOS keeps its row (fed its
        last token, output ignored) until the group is done.  Same arithmetic per sequence as generate(p); the batch-b decode
        step runs on the dense path and batch-1 on the persistent path, so logits agree to the kernel tolerance (3e-3), not
        bitwise.  Returns one id list per prompt, in request order."""
        out = [None] * len(prompts)
        groups: dict = {}
        for i, p in enumerate(prompts):
            groups.setdefault(len(p), []).append(i)
        for idxs in groups.values():
            for k in range(0, len(idxs), max_batch):
                chunk = idxs[k:k + max_batch]
                for i, toks in zip(chunk, self._generate_group([prompts[i] for i in chunk], max_tokens, temperature)):
                    out[i] = toks
        return out

    def _generate_group(self, prompts, max_tokens: int, temperature: float):
        b = len(prompts)
        self.cache = self.model.initialize_cache()
        processors = [LogitsProcessor(0, float(np.float32(temperature))) for _ in range(b)]
        ids = np.asarray(prompts, dtype=np.uint32).reshape(b, -1)
        pos = 0
        logits = self.model.forward(ids, pos, self.cache)
        pos += ids.shape[1]
        outs = [[] for _ in range(b)]
        done = [False] * b
        nxt = np.ascontiguousarray(ids[:, -1:])
        for _ in range(max_tokens):
            rows = np.asarray(logits).reshape(b, -1)
            for i in range(b):
                if done[i]:
                    continue
                tok = processors[i].sample(rows[i])
                if self.eos_token_id is not None and tok == self.eos_token_id:
                    done[i] = True                                       # break before emitting, for this sequence only
                    continue
                outs[i].append(tok)
                nxt[i, 0] = tok
            if all(done):
                break
            logits = self.model.forward(nxt, pos, self.cache)
            pos += 1
        return outs


class ContinuousBatcher:
    """Continuous batching above fl_forward_slots.  The reference serialises chat requests at batch 1
    under one mutex (api/chat.rs:206-208); here up to `max_batch` requests of ANY lengths share the decode steps: a request is
    admitted into a free sequence slot as soon as one exists (its prompt is prefilled alone, [1, T]), every step then advances all
    running requests by one token in ONE ragged forward ([n, 1], per-slot KV lengths and RoPE positions), and a request that
    hits EOS or its token budget frees its slot for the next waiting one.  Per request the arithmetic is that of
    Model.generate: its own LogitsProcessor seeded 0 (mod.rs:373-374), EOS break before emitting (mod.rs:431-436), and the
    adapter's position rule -- Llama: the caller's position; Mistral / Qwen2: +1 per CALL (mistral.rs:234, qwen.rs:143).
    `cache` needs forward_slots(slots, ids, rope_offsets) -> [n, V], slot_reset(slot): a DeviceCache, or a stand-in in tests."""

    def __init__(self, model, max_batch: int = 8, eos_token_id: int | None = 2, cache=None, prefill_chunk: int | None = None):
        """prefill_chunk (caches with forward_ragged, i.e. layered models): prompts are fed in portions of at most that many tokens
        and every step is ONE mixed batch -- the next portion of each request still reading its prompt beside the single new token of
        each request already decoding.  None: a prompt is prefilled alone in one call, then decoded in the shared steps."""
        self.model, self.max_batch, self.eos_token_id = model, max_batch, eos_token_id
        self.prefill_chunk = prefill_chunk
        # the Mistral/Qwen2 adapters' offset rule (+1 per call); Llama and the layered decoder take true positions
        self.position_per_call = getattr(model, "position_per_call", getattr(model, "arch", "llama") != "llama")
        if cache is not None:
            self.cache = cache
        elif hasattr(model, "new_device_cache"):
            self.cache = model.new_device_cache(max_batch)
        else:
            self.cache = DeviceCache(model.dev, max_batch, model._capacity())
        self.steps = 0          # ragged decode forwards issued (tests / stats)

    def generate(self, prompts, max_tokens: int, temperature: float = 0.0):
        """-> one id list per prompt, in request order."""
        if self.prefill_chunk and hasattr(self.cache, "forward_ragged"):
            return self._generate_mixed(prompts, max_tokens, temperature)
        out = [[] for _ in prompts]
        waiting = list(range(len(prompts)))[::-1]
        free = list(range(self.max_batch))[::-1]
        running = {}            # slot -> [request, next RoPE position, LogitsProcessor, token to feed]
        if max_tokens <= 0:
            return out

        def take(logits_row, req, slot, state):
            """sample -> EOS / budget -> either keep the slot running or free it"""
            tok = state[2].sample(logits_row)
            if self.eos_token_id is not None and tok == self.eos_token_id:
                done = True
            else:
                out[req].append(tok)
                state[3] = tok
                done = len(out[req]) >= max_tokens
            if done:
                running.pop(slot, None)
                self.cache.slot_reset(slot)
                free.append(slot)
            else:
                running[slot] = state

        while waiting or running:
            while waiting and free:                                   # admit: one prompt at a time, alone in its forward
                req, slot = waiting.pop(), free.pop()
                ids = np.asarray(prompts[req], dtype=np.uint32).reshape(1, -1)
                logits = self.cache.forward_slots([slot], ids, [0])
                state = [req, 1 if self.position_per_call else ids.shape[1], LogitsProcessor(0, float(np.float32(temperature))), 0]
                take(np.asarray(logits)[0].reshape(-1), req, slot, state)
            if not running:
                continue
            slots = sorted(running)
            ids = np.array([[running[s][3]] for s in slots], dtype=np.uint32)
            logits = np.asarray(self.cache.forward_slots(slots, ids, [running[s][1] for s in slots]))
            self.steps += 1
            for i, s in enumerate(slots):
                st = running[s]
                st[1] += 1
                take(logits[i].reshape(-1), st[0], s, st)
        return out


    def _generate_mixed(self, prompts, max_tokens: int, temperature: float):
        """Mixed steps: a request takes a free slot as soon as there is one; each step carries, per running request, either the next
        portion of its prompt (at most prefill_chunk tokens) or its one new token.  Sampling, EOS and the token budget are those of
        generate(); a finished request gives its slot (pages and state) back."""
        out = [[] for _ in prompts]
        if max_tokens <= 0:
            return out
        waiting = list(range(len(prompts)))[::-1]
        free = list(range(self.max_batch))[::-1]
        running = {}            # slot -> [request, prompt tokens fed, LogitsProcessor, token to feed]
        while waiting or running:
            while waiting and free:
                req, slot = waiting.pop(), free.pop()
                running[slot] = [req, 0, LogitsProcessor(0, float(np.float32(temperature))), None]
            slots = sorted(running)
            toks, want = [], []
            for s in slots:
                req, fed, _, nxt = running[s]
                prompt = prompts[req]
                if fed < len(prompt):
                    part = list(prompt[fed:fed + self.prefill_chunk])
                    running[s][1] = fed + len(part)
                    toks.append(part)
                    want.append([len(part) - 1] if running[s][1] == len(prompt) else [])
                else:
                    toks.append([nxt])
                    want.append([0])
            logits = np.asarray(self.cache.forward_ragged(slots, toks, want))
            self.steps += 1
            row = 0
            for s, w in zip(slots, want):
                if not w:
                    continue
                st = running[s]
                tok = st[2].sample(logits[row].reshape(-1))
                row += 1
                if self.eos_token_id is not None and tok == self.eos_token_id:
                    done = True
                else:
                    out[st[0]].append(tok)
                    st[3] = tok
                    done = len(out[st[0]]) >= max_tokens
                if done:
                    running.pop(s)
                    self.cache.slot_reset(s)
                    free.append(s)
        return out


# --------------------------------------------------------------------------------------------------------------------
# EmbeddingModel (models/embeddings.rs:17-38) -- BERT / MiniLM sentence encoder
# --------------------------------------------------------------------------------------------------------------------
@dataclass
class BertConfig:
    """models/embeddings.rs:46-54 (+ the vocabulary size the reference takes from the tokenizer, :301-306)."""
    hidden_size: int = 384
    num_attention_heads: int = 12
    num_hidden_layers: int = 6
    intermediate_size: int = 1536
    max_position_embeddings: int = 512
    layer_norm_eps: float = 1e-12
    vocab_size: int = 30522


class MiniLMModel:
    """MiniLMModel (models/embeddings.rs:245-447) after tokenisation: `embed_ids` takes the token ids (and the tokenizer's
    attention mask) and returns what EmbeddingModel::embed returns: the mean-pooled, L2-normalised f32 vector(s)."""
    family, architectures = "bert", ("BertModel", "RobertaModel", "DebertaModel")

    def __init__(self, config: BertConfig, tensors: dict | None, device: int = 0, model_id: str = "sentence-transformers/all-MiniLM-L6-v2",
                 random_seed=None, std: float = 0.02):
        c = FlConfig()
        c.arch = _lib.FL_ARCH["bert"]
        c.hidden_size, c.intermediate_size, c.vocab_size = config.hidden_size, config.intermediate_size, config.vocab_size
        c.num_hidden_layers, c.num_attention_heads = config.num_hidden_layers, config.num_attention_heads
        c.num_key_value_heads = config.num_attention_heads
        c.max_position_embeddings = config.max_position_embeddings
        c.norm_eps = config.layer_norm_eps
        c.rope_theta, c.tp_rank, c.tp_size = 0.0, 0, 1
        self.config, self._model_id = config, model_id
        self.dev = DeviceModel(c, device)
        if tensors is None:
            self.dev.random_init(0 if random_seed is None else random_seed, std)
        else:
            for name, arr in tensors.items():
                self.dev.put_tensor(name, np.asarray(arr, dtype=np.float32))
        self.dev.finalize()

    @classmethod
    def get_family(cls) -> str:
        return cls.family

    @classmethod
    def supports_architecture(cls, architecture: str) -> bool:
        return architecture in cls.architectures

    def model_id(self) -> str:
        return self._model_id

    def embedding_size(self) -> int:
        return self.config.hidden_size          # the reference hard-codes 384 (embeddings.rs:453-455)

    def embed_ids(self, ids: np.ndarray, mask: np.ndarray | None = None) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if ids.ndim == 1:
            ids = ids[None]
        b, t = ids.shape
        out = np.empty((b, self.config.hidden_size), dtype=np.float32)
        mptr = None
        if mask is not None:
            mask = np.ascontiguousarray(mask, dtype=np.uint32).reshape(b, t)
            mptr = mask.ctypes.data_as(C.c_void_p)
        _lib.check(self.dev.lib.fl_embed(self.dev.h, ids.ctypes.data_as(C.c_void_p), mptr, b, t, out.ctypes.data_as(C.c_void_p)))
        return out

    def embed_many(self, sentences, max_batch: int = 256) -> np.ndarray:
        """`input: [String]` batching (the reference takes one string per request, api/embeddings.rs:11-15).
        Exact by construction: the reference's attention applies NO mask (embeddings.rs:155-159) and a lone sentence has an
        all-ones mask, so padding would change results; sentences of EQUAL token length are therefore grouped into one [b, t]
        call each (no padding) and the rows scattered back in request order.  Returns f32 [len(sentences), hidden]."""
        out = np.empty((len(sentences), self.config.hidden_size), dtype=np.float32)
        groups: dict = {}
        for i, s in enumerate(sentences):
            groups.setdefault(len(s), []).append(i)
        for idxs in groups.values():
            for k in range(0, len(idxs), max_batch):
                chunk = idxs[k:k + max_batch]
                out[chunk] = self.embed_ids(np.asarray([sentences[i] for i in chunk], dtype=np.uint32))
        return out

    def embed_ids_timed(self, ids: np.ndarray, repeats: int):
        """-> (embeddings, device ms for `repeats` device-resident encoder passes over the uploaded batch)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        b, t = ids.shape
        out = np.empty((b, self.config.hidden_size), dtype=np.float32)
        ms = C.c_float()
        _lib.check(self.dev.lib.fl_embed_timed(self.dev.h, ids.ctypes.data_as(C.c_void_p), None, b, t, out.ctypes.data_as(C.c_void_p),
                                               repeats, C.byref(ms)))
        return out, ms.value

    def compute_similarity(self, ids1, ids2) -> float:
        """EmbeddingModel::compute_similarity default impl (embeddings.rs:22-37): cosine of the two embeddings."""
        v1, v2 = self.embed_ids(ids1)[0], self.embed_ids(ids2)[0]
        return float(np.dot(v1, v2) / (np.linalg.norm(v1) * np.linalg.norm(v2)))
