// Layered decoders (FL_ARCH_NIFUNEX, FL_ARCH_ROFETAR, FL_ARCH_TOZARAX, FL_ARCH_MEDULORN): model / cache objects shared by fl_layered.cu and
// fl_lib.cu.  A layer = one mixer (gated linear attention | latent attention | grouped-query attention | Mamba-2 | gated delta rule |
// lightning attention), or two of them side by side, + an optional feed-forward (dense | MoE), each wrapped by a norm before and
// after, after only (fl_stack_config.no_pre_norm), before only (no_post_norm), or a norm of the sum of stream and sublayer result
// (post_sum_norm); optionally a learned position table, an input convolution in front of every sublayer, a token shift in front of
// every mixer, a gate on every sublayer's contribution and an average over all earlier layers' outputs.  Sizes and constants
// come from fl_layer_desc / fl_stack_config; nothing is fixed per model.
#pragma once
#include <cuda.h>

#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../include/fastllm_b200.h"
#include "page_pool.hpp"
#include "runtime.cuh"

namespace fl {

struct LayeredLayerW {
    fl_layer_desc d{};
    float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr;     // [W] f32
    // mixer input projections stacked into ONE matrix [n_in, W] (one GEMM per layer):
    //   GLA:     q | k | v | g | a1        latent attention:  q | dkv   (no dkv rows when kv_from >= 0)
    //   attention:  q | k | v  (no k, v rows when kv_from >= 0)      Mamba-2:  z | x | B | C | dt      delta rule:  q | k | v | g | b | a
    // (rows padded with zeros to a multiple of 8 for the three newer mixers, so that the tensor-core GEMM's tiles fit)
    uint16_t* w_in = nullptr;
    int n_in = 0;
    int off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_a = 0, off_dkv = 0;             // row (= output column) offsets inside w_in
    int off_b = 0, off_dt = 0;          // delta rule: write strengths; Mamba-2: step sizes
    int conv_off = 0, conv_ch = 0;      // recurrent mixers with a short convolution: the convolved columns of w_in's output
    float *conv_w = nullptr, *conv_b = nullptr;                                         // [conv_ch, taps], [conv_ch] (zeros when the design has none)
    float *a_log = nullptr, *dt_bias = nullptr, *dskip = nullptr;                       // [heads]
    float *qnorm = nullptr, *knorm = nullptr;                                           // attention: [dim] ([heads * dim], [kv_heads * dim] with qk_norm_whole)
    float *bq = nullptr, *bk = nullptr, *bv = nullptr;                                  // attention with qkv_bias: [heads * dim], [kv_heads * dim], [kv_heads * vdim]
    float* sinkv = nullptr;                                                             // attention with a learned sink: [heads]
    float* decay = nullptr;                                                             // lightning attention: [heads], f32 as given
    float* shift = nullptr;                                                             // token shift: [W]
    float* router_b = nullptr;                                                          // biased router: [experts]
    float *b_gu = nullptr, *b_down = nullptr;                                           // biased dense feed-forward: [2 ff], [W]
    uint16_t* w_o = nullptr;            // [W, heads * vdim]
    // GLA
    uint16_t* a2 = nullptr;             // [heads*dim, rank]
    float *a2b = nullptr, *hnorm = nullptr;                                              // [heads*dim], [vdim]
    // latent attention
    float* dkv_norm = nullptr;          // [kv_rank]
    uint16_t* uk_t = nullptr;           // [heads][kv_rank, dim]: W_uk per head, transposed (q absorbs it: q~ = W_uk[h]^T q)
    uint16_t* uv = nullptr;             // [heads * vdim, kv_rank]
    int kv_owner = -1;                  // layer whose cache this layer reads (itself when it projects its own)
    int kv_index = -1;                  // index of that cache among the model's latent caches
    int rope_index = -1;                // index into the model's distinct rotary tables
    int gla_index = -1;                 // index among the model's recurrent layers (GLA, Mamba-2, delta rule)
    // feed-forward: groups 0..E-1 = experts (or the one dense block), `shared` separate
    uint16_t *w_gu = nullptr, *w_down = nullptr;        // [groups][2 ff, W] (gate rows then up rows), [groups][W, ff]
    uint16_t *s_gu = nullptr, *s_down = nullptr;        // shared expert
    float *router = nullptr, *shared_gate = nullptr;    // [experts, W], [W] f32
    // serving precision: TMA descriptors of the matrices whose shapes admit the tensor-core GEMM (tc_* says which)
    CUtensorMap tm_in{}, tm_o{}, tm_gu{}, tm_down{}, tm_sgu{}, tm_sdown{};
    bool tc_in = false, tc_o = false, tc_gu = false, tc_down = false, tc_sgu = false, tc_sdown = false;
    bool tc_moe = false;                               // experts: tm_gu / tm_down cover the stacked matrices (grouped GEMM, few rows),
    std::vector<CUtensorMap> tm_egu, tm_edown;         //   these one expert each (every expert over all rows, many rows)
    float* route_corr = nullptr;        // sigmoid router: [experts] added to the scores for the choice only
    // a second mixer beside this one: its rows follow this mixer's inside w_in (its offsets are absolute), it has its own w_o,
    // cache / state indices and side tables; nothing but the mixer fields of it is used
    std::shared_ptr<LayeredLayerW> side;
    float *pair_wa = nullptr, *pair_wb = nullptr;      // [W] each: plain norm weights of the two mixers' outputs
    // stack options
    float *canon1 = nullptr, *canon2 = nullptr;        // [W, taps] input convolutions of the mixer / the feed-forward
    uint16_t *rg1 = nullptr, *rg2 = nullptr;           // [W, W] gates of the two sublayers' contributions
    float *rg1b = nullptr, *rg2b = nullptr;            // [W]
    float* dwa = nullptr;                              // [layer index + 2] weights of the depth average
    CUtensorMap tm_rg1{}, tm_rg2{};
    bool tc_rg1 = false, tc_rg2 = false;
    int canon_index = -1;               // index among the layers' input-convolution states
};

struct RopeSpec {                       // one distinct rotary configuration (tables are built per cache: they depend on max_seq)
    int dims = 0;
    double base = 0;
    float yarn_factor = 0, yarn_original = 0, yarn_fast = 0, yarn_slow = 0;
    int scaling = 0;                    // fl_rot_scaling
    bool operator==(const RopeSpec& o) const {
        return dims == o.dims && base == o.base && yarn_factor == o.yarn_factor && yarn_original == o.yarn_original &&
               yarn_fast == o.yarn_fast && yarn_slow == o.yarn_slow && scaling == o.scaling;
    }
};

struct LayeredModel {
    fl_stack_config cfg{};
    int W = 0, V = 0, L = 0;
    bool f32 = false;                   // compute_dtype == FL_DTYPE_F32
    std::vector<LayeredLayerW> layers;
    std::vector<RopeSpec> ropes;
    std::vector<const LayeredLayerW*> kv_layers, gla_layers;   // mixers that own a paged cache (latent, or keys | values) / a recurrent state
    DevBuf<uint8_t> slab;
    uint16_t *embed = nullptr, *head = nullptr, *pos = nullptr;    // pos: [max_positions, W] learned position vectors (or nullptr)
    float* final_norm = nullptr;
    CUtensorMap tm_head{};
    bool tc_head = false;
    std::set<std::string> have;
    std::vector<std::string> expected;
    int ignored = 0;
    bool finalized = false;
    uint64_t weight_bytes = 0;
    // widest sizes over the layers (workspace planning)
    int max_in = 0, max_hv = 0, max_hd = 0, max_hc = 0, max_ff = 0, max_top = 0, max_experts = 0, max_cv = 0, max_heads = 0, max_av = 0;    // max_av: widest value head of a grouped-query attention layer
    std::mutex mu;
};

// Per-cache state of a layered model: latent-cache pools, recurrent-state slots, rotary tables, step tables, workspace.
struct LayeredCache {
    PagePool pool;
    bool f32 = false;
    std::vector<void*> kv_pool;         // per paged cache: [pages][64][kv_rank + rot_dim] or [pages][64][kv_heads * (dim + vdim)] (float or bf16)
    std::vector<DevBuf<uint8_t>> kv_store;
    std::vector<DevBuf<float>> gla_state;          // per recurrent layer: [slots][heads][dim | state][vdim]
    std::vector<DevBuf<float>> conv_state;         // per recurrent layer: [slots][taps - 1][conv_ch] (empty without a convolution)
    std::vector<DevBuf<float>> canon_state;        // input convolutions: per layer [2 sublayers][slots][taps - 1][W]
    std::vector<DevBuf<float>> shift_state;        // token shift: per layer [slots][W], the mixer input of the slot's last position
    std::vector<DevBuf<float>> rope_cos, rope_sin; // per RopeSpec: [max_seq][dims/2]
    DevBuf<int> page_table;             // [slots][pages_per_slot]
    DevBuf<int> step_tab;               // per-step integer tables (see StepTab in fl_layered.cu)
    PinnedBuf<int> h_step_tab;
    size_t tab_cap = 0;
    // workspace for `rows` tokens of a step
    size_t rows = 0, want_cap = 0;
    DevBuf<float> x, h, y, proj, la, u, go, qa, ol, gu, act, eo, sh_gu, sh_act, sh_o, route_w, sgate, hf, logits;
    DevBuf<float> hc, gz, y2, xs;       // convolved sublayer input; gate pre-activations; the second mixer's projected output;
                                        // xs [L + 1][rows][W]: the embedding output and every layer's own result (depth average)
    DevBuf<float> cv, rs;               // recurrent mixers: convolved + activated columns [rows, max_cv]; per-head (decay, strength) [rows, 2 heads]
    DevBuf<int> route_sel, pair_row, pair_of, grp_off;
    PinnedBuf<float> h_logits;
    // serving precision: hi/lo halves of the activations that feed tensor-core GEMMs, and the split-K slices of their outputs
    DevBuf<uint16_t> h_hi, h_lo, u_hi, u_lo, act_hi, act_lo, hf_hi, hf_lo;
    DevBuf<float> gemm_out;
    DevBuf<uint16_t> gx_hi, gx_lo, ga_hi, ga_lo;        // grouped expert GEMMs: gathered inputs / activations, [experts * cap] rows
    DevBuf<int> grp_cnt;
    // tensor-core latent attention of long portions: gathered keys, their transpose, Q / P operand halves, the score block
    DevBuf<uint16_t> at_kc, at_kct, at_qhi, at_qlo, at_phi, at_plo;
    DevBuf<float> at_part;              // grouped-query attention with key splits: partial (max, sum, values) per (row, head, split)
    DevBuf<float> at_s, at_o;           // at_o: grouped-query attention, the value GEMMs' outputs per key/value head before they are interleaved
};

void layered_build(LayeredModel& m, const fl_layer_desc* layers);
void layered_put_tensor(LayeredModel& m, const char* name, int dtype, const int64_t* shape, int rank, const void* host);
void layered_random_init(LayeredModel& m, uint64_t seed, float stdv);
void layered_finalize(LayeredModel& m);

}  // namespace fl

struct fl_cache;
namespace fl {
void layered_cache_create(fl_cache& c, int max_slots, int max_seq, int pool_tokens);
// one step of a mixed batch; logits of the wanted rows land in c.ly->h_logits (host, pinned) after the stream is synchronised
void layered_forward(fl_cache& c, const int* slots, const int* counts, int n, const uint32_t* ids, const int* want, int n_want);
void layered_slot_reset(fl_cache& c, int slot);
void layered_cache_reset(fl_cache& c);
}  // namespace fl
