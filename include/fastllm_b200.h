/* fastllm_b200 — C ABI of the B200-native transformer forward pass that slots in under fastllm's
 * trait-based model API (the L2->L0 boundary of SURVEY.md section 1 / section 8b).
 *
 * Every entry point is `extern "C"`, takes plain pointers/sizes, returns 0 on success and a negative
 * fl_status on failure; the message for the calling thread's last failure is fl_last_error().  Nothing
 * throws or aborts across this boundary.  The library owns all device memory (weights, paged KV cache,
 * workspaces), its own CUDA stream per cache, and the NCCL communicator.  There is no CPU fallback.
 *
 * Reference interface each group replaces (paths under /root/reference/src):
 *   fl_model_create / fl_model_put_tensor / fl_model_finalize
 *        <- ModelInitializer::initialize_model(&Config, HashMap<String,Tensor>, DType, &Device)
 *           models/model_initializer.rs:10-17; called from providers/huggingface/huggingface.rs:135;
 *           bodies models/llama.rs:98-123, models/mistral.rs:160-200, models/qwen.rs:93-117,
 *           and MiniLMModel::new models/embeddings.rs:257-339 (BERT family)
 *   fl_model_clone            <- `M: Clone` required by the streaming path, models/mod.rs:155,181,207
 *   fl_cache_create / reset   <- ModelInitializer::initialize_cache models/model_initializer.rs:19
 *                                (llama.rs:125-145, mistral.rs:202-204, qwen.rs:119-121) and
 *                                ModelCache::reset models/cache.rs:5-10; Mistral/Qwen2 `clear_kv_cache`
 *                                at offset 0 (mistral.rs:218-221, qwen.rs:138-140)
 *   fl_forward                <- ModelInitializer::forward(&self, &Tensor (u32 [b,t]), usize pos, &mut Cache)
 *                                models/model_initializer.rs:21 (llama.rs:147-149, mistral.rs:206-236,
 *                                qwen.rs:123-145); returns the last-position logits as f32 [b, V]
 *   fl_forward_greedy         <- forward + LogitsProcessor arg-max of models/mod.rs:421-428 fused on device
 *                                (ties resolve to the LAST index, as candle's max_by(total_cmp) does)
 *   fl_sampler_* / fl_forward_sample
 *                             <- candle's LogitsProcessor as the generate loops build and call it:
 *                                LogitsProcessor::new(Default::default(), Some(temperature as f64), None)
 *                                models/mod.rs:157-158,373-374 and logits_processor.sample(&last_logits)
 *                                models/mod.rs:308-310,425-428 (arg-max below 1e-7, else soft-max + WeightedIndex
 *                                over rand 0.8's StdRng seeded with seed_from_u64)
 *   fl_forward_slots          <- the same forward for a batch of requests of different lengths (no reference counterpart: requests
 *                                are serialised at batch 1, api/chat.rs:206-208; streams run side by side, models/mod.rs:151-175)
 *   fl_embed                  <- EmbeddingModel::embed models/embeddings.rs:397-447 after tokenisation:
 *                                encoder forward + mean_pooling (:346-368) + normalize_l2 (:341-344)
 */
#ifndef FASTLLM_B200_H
#define FASTLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FL_EXPORT __attribute__((visibility("default")))
#else
#define FL_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fl_model fl_model;
typedef struct fl_cache fl_cache;
typedef struct fl_sampler fl_sampler;

typedef enum fl_status {
    FL_OK = 0,
    FL_ERR_INVALID = -1,   /* bad argument / bad config (the reference panics: mistral.rs:109-127, models/config.rs:20-54) */
    FL_ERR_CUDA = -2,      /* CUDA runtime/driver error; the handle is poisoned */
    FL_ERR_STATE = -3,     /* call out of order (e.g. forward before finalize, cache full) */
    FL_ERR_NCCL = -4,
    FL_ERR_UNSUPPORTED = -5
} fl_status;

typedef enum fl_arch {
    FL_ARCH_LLAMA = 0,     /* LlamaForCausalLM          (models/llama.rs)   */
    FL_ARCH_MISTRAL = 1,   /* MistralForCausalLM        (models/mistral.rs) */
    FL_ARCH_QWEN2 = 2,     /* Qwen2ForCausalLM, qkv bias (models/qwen.rs)    */
    FL_ARCH_MIXTRAL = 3,   /* MixtralForCausalLM top-k MoE (no reference path; candle mixtral.rs) */
    FL_ARCH_BERT = 4,      /* BertModel encoder         (models/embeddings.rs) */
    FL_ARCH_NIFUNEX = 5,   /* layered decoder described by fl_layer_desc (no reference path): gated-linear-attention and windowed
                              latent-attention mixers, dense / mixture-of-experts feed-forward, a norm before and after each sublayer */
    FL_ARCH_ROFETAR = 6,   /* layered decoder (no reference path): grouped-query attention with a softmax sink, Mamba-2 and gated-delta-rule
                              mixers, biased gelu feed-forward; only the OUTPUT of a sublayer is normed (fl_stack_config.no_pre_norm) */
    FL_ARCH_TOZARAX = 7,   /* layered decoder (no reference path): learned positions; pre-normed sublayers that read their input through a
                              short causal convolution, gate their contribution and average over all earlier layers' outputs; two mixers
                              side by side (windowed attention without rotation | gated delta rule); sigmoid-routed squared-relu experts */
    FL_ARCH_MEDULORN = 8   /* layered decoder (no reference path): x <- norm(alpha x + sub(x)) with one number as the norm's weight
                              (fl_stack_config.post_sum_norm); mixers read x through a token shift; chunk-masked attention with biased
                              projections | sliding-window attention with kept first tokens and a learned sink beside lightning attention;
                              relu-gated dense feed-forward or clamped-swish experts with a biased router; scaled embedding, capped logits */
} fl_arch;

typedef enum fl_dtype { FL_DTYPE_F32 = 0, FL_DTYPE_BF16 = 1, FL_DTYPE_F16 = 2 } fl_dtype;

/* Mirrors the fields the reference adapters read from config.json
 * (llama.rs:17-29, mistral.rs:78-91, models/config.rs:5-18, models/embeddings.rs:46-54). */
typedef struct fl_config {
    int32_t arch;                      /* fl_arch */
    int32_t hidden_size;
    int32_t intermediate_size;
    int32_t vocab_size;
    int32_t num_hidden_layers;
    int32_t num_attention_heads;
    int32_t num_key_value_heads;       /* 0 => num_attention_heads */
    int32_t max_position_embeddings;   /* RoPE table length (causal LMs) / position table rows (BERT) */
    int32_t sliding_window;            /* Mistral/Qwen2 prefill mask: key j banned when j + sw < i; <=0 => none */
    int32_t qkv_bias;                  /* Qwen2 */
    int32_t num_local_experts;         /* Mixtral */
    int32_t num_experts_per_tok;       /* Mixtral */
    float norm_eps;                    /* rms_norm_eps, or layer_norm_eps for BERT layers (embeddings LN is 1e-12) */
    double rope_theta;
    int32_t tp_rank;                   /* tensor-parallel rank / size of THIS process (1 process per GPU) */
    int32_t tp_size;                   /* 0 or 1 => no tensor parallelism (Mixtral: the same two fields are the expert-parallel rank / size) */
    int32_t ep_dp_attention;           /* Mixtral, tp_size > 1: 1 => sequences are data-parallel (every rank is called with ITS slice of the batch,
                                          same [b, t] shape on every rank) and tokens travel to the experts and back by all-to-all;
                                          0 => every rank is called with the whole batch (attention replicated, expert outputs all-reduced) */
    int32_t reserved[5];
} fl_config;

/* ---- layered models: every layer names its own mixer and feed-forward (no reference counterpart) ----------------------------
 * A layer is  x += norm_b(mixer(norm_a(x)));  x += norm_d(ffn(norm_c(x)))  with RMS norms with a zero-centred weight
 * (x / sqrt(mean x^2 + eps) * (1 + w)).  Mixers:
 *   FL_MIXER_GLA          gated linear attention: per head a [dim, vdim] f32 state S <- diag(alpha) S + k v^T, o = S^T q with a
 *                         per-key-channel decay alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau) through a rank-`decay_rank` bottleneck;
 *                         o is RMS-normed per head, gated by silu(W_g h) and projected.  The state lives in a per-sequence slot.
 *   FL_MIXER_LATENT_ATTN  attention over a shared compressed key/value: the cache holds per token a `kv_rank` latent (RMS-normed)
 *                         and ONE rotated `rot_dim` key part; heads expand keys / values from the latent (W_uk, W_uv).  Interleaved
 *                         rotary embedding with optional YaRN frequency scaling, sliding window (`window` keys, 0 = none), plain
 *                         softmax with the given `scale`.  kv_from >= 0: the layer reads layer kv_from's cached latent instead of
 *                         projecting its own.
 *   FL_MIXER_ATTN         grouped-query softmax attention over a paged key/value cache: `heads` query heads share `kv_heads` key/value
 *                         heads (query head h reads key/value head h / (heads / kv_heads)); queries and keys are RMS-normed per head
 *                         (one weight of `dim` entries for all heads) and then turned by a rotary embedding on their first rot_dims
 *                         channels (pairs (i, i + rot_dims/2) when rot_halves, else (2i, 2i+1)); score = q.k * scale, optionally
 *                         squashed to softcap * tanh(score / softcap); `sink` adds 1 to the softmax denominator (a valueless key of
 *                         score 0).  window as for latent attention.  kv_from >= 0: the layer reads layer kv_from's cached keys and
 *                         values (as cached: normed and rotated) and projects only queries.
 *   FL_MIXER_MAMBA2       Mamba-2 state-space layer: W_in h = [z | x | B | C | dt] (inner = heads * vdim, `groups` x `state` for B and
 *                         C); x|B|C pass a causal per-channel convolution of `conv` taps with bias, then silu; dt = softplus(dt + bias);
 *                         per head an f32 state S [state, vdim]: S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; y * silu(z) is
 *                         RMS-normed in `norm_groups` equal parts, scaled by a weight and projected.
 *   FL_MIXER_DELTA        gated delta rule: q, k (kv_heads x dim) and v (heads x vdim) pass a bias-free causal convolution of `conv`
 *                         taps and silu; q and k become unit vectors per head (q also times dim^-1/2); beta = sigmoid(W_b h), decay
 *                         g = exp(-exp(A_log) softplus(W_a h + dt_bias)) per head; per head an f32 state S [dim, vdim]: S <- g S,
 *                         u = beta (v - S^T k), S <- S + k u^T, o = S^T q; o is RMS-normed per head, gated by silu(W_g h), projected.
 * The recurrent mixers keep, per sequence slot, the state S and the last conv - 1 inputs of every convolved channel.
 * Feed-forward (ffn_act = FL_ACT_SWISH_CLAMP): y = W_down (g * sigmoid(1.702 g) * (u + 1)), g = min(W_gate h, limit), u = clamp(W_up h,
 * -limit, limit); (ffn_act = FL_ACT_GELU_TANH): y = W_down (gelu_tanh(W_gate h) * (W_up h)); ffn_bias adds a bias to all three
 * projections; (ffn_act = FL_ACT_RELU2): y = W_down relu(W_up h)^2, no gate matrix.  Dense, or `top` of `experts` such experts
 * weighted by their renormalised softmax scores plus an optional always-on shared expert scaled by sigmoid(w_sg . h)
 * (router = FL_ROUTER_SOFTMAX); or (router = FL_ROUTER_SIGMOID_GROUPS) scores s = sigmoid(W_r h), choice scores s + correction, the
 * experts form `route_groups` equal groups of neighbours of which the `route_keep` with the largest sum of their two best choice
 * scores stay eligible, the `top` eligible experts with the largest choice scores are used with weights s (not renormalised).
 * Two mixers side by side (`beside`): both read the layer's mixer input; the layer's mixer output is half the sum of the two
 * outputs, each RMS-normed over the width with a plain weight ("l<i>.mix.left.out" / "l<i>.mix.right.out"); their tensors are
 * "l<i>.mix.left.*" / "l<i>.mix.right.*"; with `pair_sum` the output is out_scale_left * left + out_scale_right * right instead and
 * no such weights exist.
 *   FL_MIXER_LIGHTNING    lightning attention: q = silu(W_q h), k = silu(W_k h) (heads x dim), v = silu(W_v h) (heads x vdim); per head an
 *                         f32 state S [dim, vdim]: S <- decay_h S + k v^T, o = S^T q with one fixed decay per head (tensor "decay"
 *                         [heads], kept in f32 as given); the concatenated heads are RMS-normed together (plain weight "norm"
 *                         [heads * vdim]), multiplied by sigmoid(W_g h) and projected.
 * Attention masks: `window` (i - j < window), `keep_first` (keys j < keep_first stay visible whatever the window; they keep their own
 * positions) and `mask_chunk` (i and j must lie in the same block of mask_chunk positions counted from the sequence's start) combine:
 * j <= i is visible iff it passes the chunk rule and (the window rule or the kept-first rule).  sink = 2: the softmax denominator
 * gains exp(s_h) with a learned s_h per query head (tensor "sink" [heads], not scaled).  qkv_bias: "q.b" / "k.b" / "v.b" are added
 * to the projections.  qk_norm_whole: the q (and k) norm runs over all heads' channels at once with a weight of that length.
 * rot_scaling = FL_ROT_SCALE_BANDS: frequencies whose wavelength is below yarn_original / yarn_fast stay, above yarn_original /
 * yarn_slow are divided by yarn_factor, between the two blend linearly in yarn_original / wavelength; cos and sin keep magnitude 1.
 * Feed-forward (ffn_act = FL_ACT_RELU): y = W_down (relu(W_gate h) * (W_up h)).  router_bias: "mlp.router.b" is added to the router
 * logits.  shared_plain: the shared expert's output is added as it is (no "mlp.shared.sg"). */
typedef enum fl_mixer_kind { FL_MIXER_GLA = 0, FL_MIXER_LATENT_ATTN = 1, FL_MIXER_ATTN = 2, FL_MIXER_MAMBA2 = 3, FL_MIXER_DELTA = 4, FL_MIXER_LIGHTNING = 5 } fl_mixer_kind;
typedef enum fl_ffn_kind { FL_FFN_NONE = 0, FL_FFN_DENSE = 1, FL_FFN_MOE = 2 } fl_ffn_kind;
typedef enum fl_ffn_act { FL_ACT_SWISH_CLAMP = 0, FL_ACT_GELU_TANH = 1, FL_ACT_RELU2 = 2, FL_ACT_RELU = 3 } fl_ffn_act;
typedef enum fl_rot_scaling { FL_ROT_SCALE_YARN = 0, FL_ROT_SCALE_BANDS = 1 } fl_rot_scaling;
typedef enum fl_router_kind { FL_ROUTER_SOFTMAX = 0, FL_ROUTER_SIGMOID_GROUPS = 1 } fl_router_kind;

typedef struct fl_layer_desc {
    int32_t mixer;                     /* fl_mixer_kind */
    int32_t heads, dim, vdim;          /* per head: query/key channels (unrotated part for latent attention), value channels */
    int32_t decay_rank;                /* GLA: rows of the decay bottleneck */
    float tau;                         /* GLA: decay temperature */
    int32_t rot_dim, kv_rank;          /* latent attention: rotated channels per head / latent width */
    int32_t kv_from;                   /* latent attention: layer whose cached latent is read, -1 = its own */
    int32_t window;                    /* latent attention: position i sees j with 0 <= i - j < window; 0 = every earlier key */
    int32_t rot_dims;                  /* leading channels of the rotated part that turn (pairs 2i, 2i+1) */
    double rot_base;
    float scale;                       /* multiplies the scores */
    float yarn_factor;                 /* 0 = plain rotary; else YaRN with the next three */
    float yarn_original, yarn_fast, yarn_slow;
    int32_t ffn;                       /* fl_ffn_kind */
    int32_t ff;                        /* dense: hidden width; MoE: hidden width of one expert */
    float limit;
    int32_t experts, top;              /* MoE */
    int32_t shared_ff;                 /* MoE: hidden width of the shared expert, 0 = none */
    float shared_limit;
    int32_t kv_heads;                  /* attention / delta rule: key (and query, for the delta rule) heads; 0 = heads */
    int32_t conv;                      /* Mamba-2 / delta rule: taps of the short causal convolution */
    int32_t state, groups, norm_groups;/* Mamba-2: state size per head, B / C groups, parts of the gated output norm */
    float softcap;                     /* attention: score <- softcap * tanh(score / softcap); 0 = none */
    int32_t sink;                      /* attention: 1 = one is added to the softmax denominator; 2 = exp(sink_h), a learned number per head */
    int32_t rot_halves;                /* attention: 1 = rotary pairs are (i, i + rot_dims / 2), 0 = (2i, 2i + 1) */
    int32_t ffn_act, ffn_bias;         /* feed-forward: fl_ffn_act; dense: 1 = gate / up / down carry biases */
    int32_t no_qk_norm;                /* attention: 1 = queries and keys are used as projected (no per-head norm, no norm tensors) */
    int32_t beside;                    /* 1 = the NEXT descriptor of the array describes a second mixer of this layer (its mixer fields only;
                                          it counts as no layer of its own); attention or delta rule, each with its own cache / state */
    int32_t router;                    /* MoE: fl_router_kind */
    int32_t route_groups, route_keep;  /* FL_ROUTER_SIGMOID_GROUPS: groups of neighbouring experts / groups that stay eligible */
    int32_t qkv_bias;                  /* attention: 1 = the q, k and v projections carry biases */
    int32_t qk_norm_whole;             /* attention: 1 = q and k are normed over all their heads' channels at once (weights of that length) */
    int32_t mask_chunk;                /* attention: > 0 = a position sees only the keys of its own block of this many positions */
    int32_t keep_first;                /* attention with a window: the first keep_first keys of the sequence stay visible */
    int32_t rot_scaling;               /* fl_rot_scaling: how yarn_factor / yarn_original / yarn_fast / yarn_slow change the frequencies */
    float out_scale;                   /* mixers side by side with pair_sum: this mixer's share of the sum */
    int32_t pair_sum;                  /* beside: 1 = the layer's mixer output is the out_scale-weighted sum of the two mixers' outputs */
    int32_t router_bias;               /* MoE, FL_ROUTER_SOFTMAX: 1 = the router logits carry a bias */
    int32_t shared_plain;              /* MoE: 1 = the shared expert is not gated */
    int32_t reserved[2];
} fl_layer_desc;

typedef struct fl_stack_config {
    int32_t arch;                      /* FL_ARCH_NIFUNEX */
    int32_t vocab, width, n_layers;
    float norm_eps;
    int32_t compute_dtype;             /* FL_DTYPE_BF16: bf16 weights on the tensor-core path, bf16 cache; FL_DTYPE_F32: every product
                                          and the cache in true 32-bit (weights are still stored as the bf16 values they were given) */
    int32_t norm_plain;                /* 0: the layer norms and the final norm scale by (1 + w);  1: by w */
    int32_t no_pre_norm;               /* 0: x += norm_b(sub(norm_a(x)));  1: x += norm(sub(x)) -- sublayers read the residual stream itself
                                          and "l<i>.norm1" / "l<i>.norm2" name the norms of the mixer's / feed-forward's output */
    int32_t no_post_norm;              /* 1: x += sub(norm_a(x)) -- a sublayer's result joins the stream as it is (needs pre-norms) */
    int32_t max_positions;             /* > 0: a learned position vector "pos" [max_positions, width] is added to the embedding */
    int32_t canon_taps;                /* > 0: every sublayer reads h + conv(h) instead of its input h, a causal per-channel convolution of
                                          this many taps ("l<i>.canon1" / "canon2" [width, taps], last column = the current token); the last
                                          taps - 1 inputs are kept per sequence slot */
    int32_t gated_residual;            /* 1: a sublayer's result is multiplied by sigmoid(W h + b) ("l<i>.rg1|rg2" [width, width], ".b"),
                                          h = the sublayer's normed input before the convolution */
    int32_t depth_avg;                 /* 1: what leaves layer i is sum_j dwa[j] X_j over X_0 = the embedding output and X_j+1 = layer j's own
                                          result, j <= i ("l<i>.dwa" [i + 2]) */
    int32_t post_sum_norm;             /* 1: x <- norm(residual_alpha x + sub(x)) -- the norm follows the sum (needs no_pre_norm; "l<i>.norm1" /
                                          "norm2" name these norms) */
    float residual_alpha;
    int32_t norm_scalar;               /* 1: every layer norm and the final norm has ONE number as its weight (a tensor of one element) */
    float embed_scale;                 /* != 0: the embedding row is multiplied by this */
    float logit_softcap;               /* > 0: logits <- cap tanh(logits / cap) */
    int32_t token_shift;               /* 1: a mixer reads h + (h_prev - h) * shift, h_prev = the previous token's mixer input of the same layer
                                          before this replacement, zeros at position 0 ("l<i>.shift" [width]); h_prev is kept per slot and layer */
    int32_t reserved[3];
} fl_stack_config;

/* ---- process / device -------------------------------------------------------------------------- */
FL_EXPORT int fl_init(int device);                               /* cudaSetDevice + one-time setup; idempotent */
FL_EXPORT const char* fl_last_error(void);                       /* thread-local, never NULL */
FL_EXPORT int fl_version(void);
FL_EXPORT int fl_device_synchronize(void);

/* ---- model (weights) --------------------------------------------------------------------------- */
FL_EXPORT int fl_model_create(const fl_config* cfg, fl_model** out);
/* A layered model: cfg->n_layers entries of `layers` (plus one more after every entry with `beside` set).  Tensors then arrive by name through fl_model_put_tensor ("embed", "head",
 * "final.norm", "l<i>.norm1|norm1b|norm2|norm2b" (no_pre_norm: "l<i>.norm1|norm2"), "l<i>.mix.*", "l<i>.mlp.*"); fl_model_finalize
 * checks that all came. */
FL_EXPORT int fl_model_create_layered(const fl_stack_config* cfg, const fl_layer_desc* layers, fl_model** out);
/* Upload one tensor by its HuggingFace name (same names VarBuilder asks for).  f32/f16 inputs are rounded to
 * bf16 (round-to-nearest-even), as VarBuilder::from_tensors(.., DType::BF16, ..) does (main.rs:120).  The host
 * buffer may be freed on return.  q/k/v and gate/up are fused and row-permuted on upload. */
FL_EXPORT int fl_model_put_tensor(fl_model* m, const char* name, int dtype, const int64_t* shape, int rank, const void* host_ptr);
/* Deterministic synthetic weights generated on the device (rule: oracle/synth.py; N(0,std^2)-like -> bf16,
 * norm weights 1.0).  Used by the benchmark instead of shipping 14-93 GB of tensors. */
FL_EXPORT int fl_model_random_init(fl_model* m, uint64_t seed, float std);
FL_EXPORT int fl_model_finalize(fl_model* m);                    /* checks every tensor arrived; builds RoPE tables */
FL_EXPORT int fl_model_clone(fl_model* m, fl_model** out);       /* shares weights (ref-counted), independent otherwise */
FL_EXPORT int fl_model_destroy(fl_model* m);
FL_EXPORT int fl_model_weight_bytes(fl_model* m, uint64_t* streamed_bytes); /* bytes one decode step must stream (no embedding table) */

/* ---- KV cache ---------------------------------------------------------------------------------- */
FL_EXPORT int fl_cache_create(fl_model* m, int max_batch, int max_seq, fl_cache** out);
/* A cache whose pages are handed out on demand: `max_slots` sequence slots (each with the recurrent state of the model's
 * stateful layers) share a pool of ceil(pool_tokens / 64) pages; a slot takes pages as it grows, up to max_seq tokens, and
 * fl_cache_slot_reset gives them back.  Layered models only (for them fl_cache_create is this with pool_tokens = max_batch x max_seq). */
FL_EXPORT int fl_cache_create_pooled(fl_model* m, int max_slots, int max_seq, int pool_tokens, fl_cache** out);
FL_EXPORT int fl_cache_pool_stats(fl_cache* c, int* pages_total, int* pages_free);
FL_EXPORT int fl_cache_reset(fl_cache* c);                       /* kv length := 0 for every sequence */
FL_EXPORT int fl_cache_kv_len(fl_cache* c, int* out);            /* tokens currently held (same for every sequence) */
FL_EXPORT int fl_cache_fill_synthetic(fl_cache* c, int batch, int kv_len, uint64_t seed); /* benchmark: pretend a kv_len-token prefill */
FL_EXPORT int fl_cache_destroy(fl_cache* c);

/* ---- forward (causal LMs) ---------------------------------------------------------------------- */
/* ids: host u32 [b, t] row-major.  rope_offset: RoPE position of ids[:,0] (explicit so the Mistral/Qwen2 adapter's
 * +1-per-call rule survives unchanged; the KV length is tracked inside the cache).  logits_host: f32 [b, vocab]. */
FL_EXPORT int fl_forward(fl_model* m, fl_cache* c, const uint32_t* ids, int b, int t, size_t rope_offset, float* logits_host);
/* Same forward, arg-max on device (last index wins ties); next_ids: host u32 [b]. */
FL_EXPORT int fl_forward_greedy(fl_model* m, fl_cache* c, const uint32_t* ids, int b, int t, size_t rope_offset, uint32_t* next_ids);
/* Device-resident greedy decode: `steps` single-token steps where step i feeds the arg-max of step i-1 (first step feeds
 * first_ids), RoPE position rope_offset+i.  One CUDA-graph launch per step, no host sync inside.  out_ids: host u32
 * [steps, b] or NULL.  elapsed_ms: CUDA-event time of the whole loop on the cache's stream, or NULL. */
FL_EXPORT int fl_decode_greedy_loop(fl_model* m, fl_cache* c, const uint32_t* first_ids, int b, size_t rope_offset, int steps,
                          uint32_t* out_ids, float* elapsed_ms);

/* ---- continuous batching: sequence slots with their own lengths -------------------------------------
 * The reference serialises requests at batch 1 under a mutex (api/chat.rs:206-208) and runs streams concurrently at batch 1 each
 * (models/mod.rs:151-175).  A cache created with max_batch > 1 holds max_batch independent sequence SLOTS; fl_forward_slots feeds
 * t new tokens to each of n distinct slots in ONE forward -- a new request's prompt (n = 1, t = prompt length) or one decode step
 * of every running request (t = 1), whatever their lengths -- with a RoPE position per row (explicit, like fl_forward's, so the
 * Mistral/Qwen2 adapters' +1-per-call rule survives per request).  logits_host: f32 [n, vocab], row i = slot slots[i].
 * A cache is driven either by the uniform calls above or by slots; fl_cache_reset switches back. */
FL_EXPORT int fl_forward_slots(fl_model* m, fl_cache* c, const int* slots, const uint32_t* ids, int n, int t, const size_t* rope_offsets,
                               float* logits_host);
/* One step of a mixed batch (layered models): sequence i of the call lives in slot slots[i] and is fed counts[i] >= 1 new tokens
 * (a portion of a prompt, or one decoded token) at the positions that follow what the slot already holds; ids holds the tokens of
 * all sequences back to back.  want[k] indexes that flattened token list: logits_host receives f32 [n_want, vocab] in that order
 * (n_want may be 0).  The result at a position does not depend on how its sequence was cut into calls or on what else is in the
 * batch, beyond rounding. */
FL_EXPORT int fl_forward_ragged(fl_model* m, fl_cache* c, const int* slots, const int* counts, int n, const uint32_t* ids,
                                const int* want, int n_want, float* logits_host);
FL_EXPORT int fl_cache_slot_reset(fl_cache* c, int slot);        /* the slot's sequence is finished: length := 0 */
FL_EXPORT int fl_cache_slot_len(fl_cache* c, int slot, int* out);

/* Diagnostics (no reference counterpart): the router's decisions in the LAST forward on this cache (Mixtral only) -- experts
 * [layers][rows][num_experts_per_tok] in pick order (MixtralSparseMoeBlock's sort, models/mixtral.rs via candle-transformers) and
 * margins [layers][rows] = softmax-probability gap between the last picked expert and the best one left out; rows = batch x t of
 * that forward.  top-k routing is discontinuous: a sharded run whose hidden state differs in the last f32 bits can pick another
 * expert where the margin is ~0, so the sharded-vs-single-GPU checks (bench.py, tests/test_tp.py) compare logits only where the
 * routing agrees and require every disagreement to sit on such a near-tie. */
FL_EXPORT int fl_cache_moe_routing(fl_cache* c, int rows, int32_t* experts, float* margins);

/* ---- sampling (host arithmetic: the reference samples on the host from every forward's logits) --- */
/* LogitsProcessor::new(seed, Some(temperature), None): temperature < 1e-7 => arg-max (IEEE total order, LAST index among
 * equal maxima); otherwise softmax(logits * (1/T as f32)) with a sequential f32 denominator, then
 * WeightedIndex<f32>::sample over StdRng::seed_from_u64(seed) (ChaCha12).  The reference always passes seed 0. */
FL_EXPORT int fl_sampler_create(uint64_t seed, double temperature, fl_sampler** out);
FL_EXPORT int fl_sampler_sample(fl_sampler* s, const float* logits_host, size_t n, uint32_t* token);
/* The arg-max rule above for every row of a host f32 [rows, n] matrix (a batch of greedy requests); tokens: host u32 [rows]. */
FL_EXPORT int fl_argmax_rows(const float* logits_host, int rows, size_t n, uint32_t* tokens);
FL_EXPORT int fl_sampler_next_u32(fl_sampler* s, uint32_t* out);  /* the generator's next raw word (known-answer tests) */
FL_EXPORT int fl_sampler_destroy(fl_sampler* s);
/* fl_forward, then sample row 0 of the logits (the generate loop only looks at logits.get(0), models/mod.rs:421); one
 * vocab*4-byte read-back, no caller-side logits buffer.  next_id: host u32 [1]. */
FL_EXPORT int fl_forward_sample(fl_model* m, fl_cache* c, const uint32_t* ids, int b, int t, size_t rope_offset, fl_sampler* s,
                                uint32_t* next_id);

/* Opt-in fast path of the same call: the soft-max weights, their prefix sums and the search run ON THE DEVICE (the sampler object
 * still owns the generator and hands over its one draw per sample, so a request's random stream is unchanged); 4 bytes travel back
 * instead of vocab * 4.  Not bit-identical to the host path by construction: the prefix sums come from a block scan, so a draw
 * within ~1e-6 (relative) of a boundary between two tokens may pick the neighbour.  The parity path is fl_forward_sample. */
FL_EXPORT int fl_forward_sample_device(fl_model* m, fl_cache* c, const uint32_t* ids, int b, int t, size_t rope_offset, fl_sampler* s,
                                       uint32_t* next_id);

/* ---- embeddings (BERT family) ------------------------------------------------------------------ */
/* ids/mask: host u32 [b, t]; mask may be NULL (all ones).  out: host f32 [b, hidden], mean-pooled and L2-normalised. */
FL_EXPORT int fl_embed(fl_model* m, const uint32_t* ids, const uint32_t* mask, int b, int t, float* out);
/* Benchmark hook: one fl_embed, then `repeats` device-resident encoder passes over the same (already uploaded) batch;
 * device_ms = CUDA-event time of those repeats on the model's stream. */
FL_EXPORT int fl_embed_timed(fl_model* m, const uint32_t* ids, const uint32_t* mask, int b, int t, float* out, int repeats, float* device_ms);

/* ---- tensor / expert parallelism (one process per GPU; the library owns the NCCL communicator) -- */
FL_EXPORT int fl_comm_unique_id(void* out_128_bytes);            /* rank 0 creates, the host side broadcasts it */
FL_EXPORT int fl_comm_init(int rank, int world, const void* unique_id_128_bytes);
/* Peer-memory exchange area of the persistent decode kernel's in-kernel all-reduce (CUDA IPC over NVLink): every rank exports
 * its buffer handle, the host side all-gathers the 64-byte handles, every rank imports all of them ([world][64] bytes). */
FL_EXPORT int fl_comm_ipc_export(void* handle_64_bytes);
FL_EXPORT int fl_comm_ipc_import(const void* handles, int world, int rank);
FL_EXPORT int fl_comm_destroy(void);

/* ---- measurement hooks (bench.py / tests) ------------------------------------------------------- */
/* Per-kernel CUDA-event profile of subsequent forwards (eager launches, events on the launching stream). */
FL_EXPORT int fl_prof_begin(void);
/* Writes a JSON array [{"kernel": name, "launches": n, "ms": total_ms, "bytes": algorithmic_bytes}, ...]. */
FL_EXPORT int fl_prof_end(char* json_out, size_t cap);
FL_EXPORT int fl_launch_count(uint64_t* kernels_launched);       /* kernels this library launched since load */

#ifdef __cplusplus
}
#endif
#endif /* FASTLLM_B200_H */
