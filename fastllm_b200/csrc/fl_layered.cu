// Layered decoders (FL_ARCH_NIFUNEX, FL_ARCH_ROFETAR, FL_ARCH_TOZARAX, FL_ARCH_MEDULORN): weight layout + ingest, pooled cache (pages of latents or keys | values +
// recurrent-state slots), and the step function for mixed batches (portions of prompts beside single decoded tokens).
#include <cmath>
#include <map>

#include "layered_model.cuh"
#include "layered_ops.cuh"
#include "model.cuh"
#include "synth.cuh"

namespace fl {

static inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }
// grouped-query attention: a launch of few (row, head) pairs splits each row's keys over up to kGqaMaxSplits blocks
constexpr int kGqaMaxSplits = 16, kGqaSplitRows = 4 * 296;
// the softmax between the two attention GEMMs keeps a row's scores in shared memory when the row has at most this many visible keys
constexpr int kSoftmaxKeep = 10240;

static float bits_to_f32(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static uint16_t f32_to_bits(float f) {
    uint32_t b;
    std::memcpy(&b, &f, 4);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((b >> 16) | 0x40u);
    return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
static float half_to_f32(uint16_t h) {
    const int e = (h >> 10) & 0x1F, m = h & 0x3FF;
    float v = e == 0 ? std::ldexp((float)m, -24) : (e == 31 ? (m ? NAN : INFINITY) : std::ldexp((float)(m + 1024), e - 25));
    return (h & 0x8000) ? -v : v;
}

// where a named tensor goes
struct LyRoute {
    enum Kind { MAT16, F32, UK_T, F32_RAW, F32_FILL } kind;     // F32_RAW: f32 input is kept bit for bit (constants of a design, not
                                                                // weights); F32_FILL: a tensor of ONE element fills rows x cols floats
    void* dst;
    int64_t rows, cols;     // shape handed over
    int heads;              // UK_T: source rows = heads * (rows / heads)
};
struct LayeredRoutes {
    std::map<std::string, LyRoute> r;
};
static std::map<const LayeredModel*, LayeredRoutes> g_routes;      // built with the model, dropped at finalize
static std::mutex g_routes_mu;

static void check_mixer(const LayeredModel& m, int i, const fl_layer_desc& d, bool second) {
    const std::string at = "layer " + std::to_string(i) + (second ? " (second mixer): " : ": ");
    FL_CHECK(d.heads >= 1 && (d.dim >= 1 || d.mixer == FL_MIXER_MAMBA2) && d.vdim >= 1, FL_ERR_INVALID, at + "heads / dim / vdim must be positive");
    if (second || d.beside)
        FL_CHECK((d.mixer == FL_MIXER_ATTN || d.mixer == FL_MIXER_DELTA || d.mixer == FL_MIXER_LIGHTNING) && d.kv_from < 0, FL_ERR_UNSUPPORTED,
                 at + "mixers side by side: attention, delta rule or lightning attention, each with its own cache");
    if (d.mixer == FL_MIXER_GLA) {
        FL_CHECK(d.decay_rank >= 1 && d.decay_rank <= 4096 && d.tau > 0.f, FL_ERR_INVALID, at + "bad decay rank / tau");
        FL_CHECK(d.dim <= 256, FL_ERR_UNSUPPORTED, at + "gated linear attention: at most 256 key channels per head");
    } else if (d.mixer == FL_MIXER_LATENT_ATTN) {
        FL_CHECK(d.kv_rank >= 1 && d.kv_rank <= 512 && d.rot_dim >= 0 && d.rot_dim <= 128, FL_ERR_UNSUPPORTED,
                 at + "latent attention: kv_rank <= 512 and rot_dim <= 128");
        FL_CHECK(d.rot_dims >= 0 && d.rot_dims <= d.rot_dim && d.rot_dims % 2 == 0, FL_ERR_INVALID, at + "rotated channels must be even and <= rot_dim");
        FL_CHECK(d.window >= 0, FL_ERR_INVALID, at + "negative window");
        if (d.kv_from >= 0) {
            FL_CHECK(d.kv_from < i, FL_ERR_INVALID, at + "kv_from must name an earlier layer");
            const fl_layer_desc& s = m.layers[d.kv_from].d;
            FL_CHECK(s.mixer == FL_MIXER_LATENT_ATTN && s.kv_from < 0 && s.kv_rank == d.kv_rank && s.rot_dim == d.rot_dim &&
                         s.rot_dims == d.rot_dims && s.rot_base == d.rot_base && s.yarn_factor == d.yarn_factor &&
                         s.yarn_original == d.yarn_original && s.yarn_fast == d.yarn_fast && s.yarn_slow == d.yarn_slow,
                     FL_ERR_INVALID, at + "kv_from must name a latent-attention layer with its own cache and the same latent / rotary sizes");
        }
    } else if (d.mixer == FL_MIXER_ATTN) {
        const int G = d.kv_heads > 0 ? d.kv_heads : d.heads;
        FL_CHECK(d.heads % G == 0, FL_ERR_INVALID, at + "heads must be a multiple of kv_heads");
        FL_CHECK(d.dim <= 256 && d.vdim <= 256, FL_ERR_UNSUPPORTED, at + "attention: at most 256 channels per head");
        FL_CHECK(d.rot_dims >= 0 && d.rot_dims <= d.dim && d.rot_dims % 2 == 0, FL_ERR_INVALID, at + "rotated channels must be even and <= dim");
        FL_CHECK(d.window >= 0 && d.softcap >= 0.f, FL_ERR_INVALID, at + "negative window / score cap");
        FL_CHECK(d.keep_first >= 0 && d.mask_chunk >= 0 && d.sink >= 0 && d.sink <= 2, FL_ERR_INVALID, at + "bad mask sizes / sink kind");
        FL_CHECK(d.rot_scaling == FL_ROT_SCALE_YARN || d.rot_scaling == FL_ROT_SCALE_BANDS, FL_ERR_INVALID, at + "unknown rotary scaling");
        FL_CHECK(!(d.qk_norm_whole && d.no_qk_norm), FL_ERR_INVALID, at + "a q/k norm over the whole projection needs the q/k norm");
        FL_CHECK(!(d.qkv_bias && d.kv_from >= 0), FL_ERR_UNSUPPORTED, at + "biased projections are built for layers with their own cache");
        if (d.kv_from >= 0) {
            FL_CHECK(d.kv_from < i, FL_ERR_INVALID, at + "kv_from must name an earlier layer");
            const fl_layer_desc& s = m.layers[d.kv_from].d;
            const int Gs = s.kv_heads > 0 ? s.kv_heads : s.heads;
            FL_CHECK(s.mixer == FL_MIXER_ATTN && s.kv_from < 0 && Gs == G && s.dim == d.dim && s.vdim == d.vdim, FL_ERR_INVALID,
                     at + "kv_from must name an attention layer with its own cache and the same key / value head sizes");
        }
    } else if (d.mixer == FL_MIXER_MAMBA2) {
        FL_CHECK(d.state >= 1 && d.state <= 256, FL_ERR_UNSUPPORTED, at + "Mamba-2: state size must be in 1..256");
        FL_CHECK(d.groups >= 1 && d.heads % d.groups == 0, FL_ERR_INVALID, at + "heads must be a multiple of groups");
        FL_CHECK(d.norm_groups >= 1 && (d.heads * d.vdim) % d.norm_groups == 0, FL_ERR_INVALID, at + "the inner width must divide into norm_groups parts");
        FL_CHECK(d.conv >= 1 && d.conv <= kMaxTaps, FL_ERR_UNSUPPORTED, at + "convolution taps must be in 1..16");
    } else if (d.mixer == FL_MIXER_DELTA) {
        const int G = d.kv_heads > 0 ? d.kv_heads : d.heads;
        FL_CHECK(d.heads % G == 0, FL_ERR_INVALID, at + "heads must be a multiple of kv_heads");
        FL_CHECK(d.dim <= 256, FL_ERR_UNSUPPORTED, at + "delta rule: at most 256 key channels per head");
        FL_CHECK(d.conv >= 1 && d.conv <= kMaxTaps, FL_ERR_UNSUPPORTED, at + "convolution taps must be in 1..16");
    } else if (d.mixer == FL_MIXER_LIGHTNING) {
        FL_CHECK(d.dim <= 256, FL_ERR_UNSUPPORTED, at + "lightning attention: at most 256 key channels per head");
    } else {
        FL_CHECK(false, FL_ERR_INVALID, at + "unknown mixer");
    }
}

static void check_layer(const LayeredModel& m, int i, const fl_layer_desc& d) {
    const std::string at = "layer " + std::to_string(i) + ": ";
    check_mixer(m, i, d, false);
    FL_CHECK(d.ffn_act == FL_ACT_SWISH_CLAMP || d.ffn_act == FL_ACT_GELU_TANH || d.ffn_act == FL_ACT_RELU2 || d.ffn_act == FL_ACT_RELU, FL_ERR_INVALID,
             at + "unknown feed-forward activation");
    FL_CHECK(!(d.ffn_act == FL_ACT_RELU && d.ffn_bias), FL_ERR_UNSUPPORTED, at + "the relu-gated feed-forward has no biases");
    FL_CHECK(d.ffn != FL_FFN_MOE || ((d.ffn_act == FL_ACT_SWISH_CLAMP || d.ffn_act == FL_ACT_RELU2) && !d.ffn_bias), FL_ERR_UNSUPPORTED,
             at + "experts use the clamped or the squared-relu activation, without biases");
    FL_CHECK(!(d.ffn_act == FL_ACT_RELU2 && d.ffn_bias), FL_ERR_UNSUPPORTED, at + "the squared-relu feed-forward has no biases");
    if (d.ffn == FL_FFN_DENSE) {
        FL_CHECK(d.ff >= 1, FL_ERR_INVALID, at + "ff must be positive");
    } else if (d.ffn == FL_FFN_MOE) {
        FL_CHECK(d.ff >= 1 && d.experts >= 1 && d.experts <= 1024 && d.top >= 1 && d.top <= d.experts && d.shared_ff >= 0, FL_ERR_INVALID,
                 at + "bad expert counts");
        FL_CHECK(d.router == FL_ROUTER_SOFTMAX || d.router == FL_ROUTER_SIGMOID_GROUPS, FL_ERR_INVALID, at + "unknown router");
        if (d.router == FL_ROUTER_SIGMOID_GROUPS) {
            FL_CHECK(d.route_groups >= 1 && d.experts % d.route_groups == 0 && d.route_keep >= 1 && d.route_keep <= d.route_groups, FL_ERR_INVALID,
                     at + "experts must divide into route_groups groups of which 1..route_groups are kept");
            FL_CHECK(d.top <= d.route_keep * (d.experts / d.route_groups), FL_ERR_INVALID, at + "the kept groups hold fewer than `top` experts");
            FL_CHECK(d.shared_ff == 0, FL_ERR_UNSUPPORTED, at + "the sigmoid router has no shared expert");
            FL_CHECK(!d.router_bias, FL_ERR_UNSUPPORTED, at + "the sigmoid router has a choice correction, not a bias");
        }
    } else {
        FL_CHECK(d.ffn == FL_FFN_NONE, FL_ERR_INVALID, at + "unknown feed-forward kind");
    }
}

void layered_build(LayeredModel& m, const fl_layer_desc* descs) {
    const fl_stack_config& c = m.cfg;
    FL_CHECK(c.arch == FL_ARCH_NIFUNEX || c.arch == FL_ARCH_ROFETAR || c.arch == FL_ARCH_TOZARAX || c.arch == FL_ARCH_MEDULORN, FL_ERR_INVALID,
             "layered models: unknown arch");
    FL_CHECK(c.vocab >= 1 && c.width >= 1 && c.n_layers >= 1 && c.n_layers <= 4096, FL_ERR_INVALID, "layered models: sizes must be positive");
    FL_CHECK(c.compute_dtype == FL_DTYPE_BF16 || c.compute_dtype == FL_DTYPE_F32, FL_ERR_INVALID, "compute_dtype must be bf16 or f32");
    FL_CHECK(!(c.no_pre_norm && c.no_post_norm), FL_ERR_INVALID, "a stack norms its sublayers' inputs, their outputs, or both");
    FL_CHECK(c.max_positions >= 0 && c.canon_taps >= 0 && c.canon_taps <= kMaxTaps, FL_ERR_INVALID, "bad position table / input convolution size");
    FL_CHECK(c.no_post_norm || !(c.gated_residual || c.depth_avg), FL_ERR_UNSUPPORTED,
             "gated contributions and the depth average are built for stacks whose sublayer results join the stream un-normed");
    FL_CHECK(!c.post_sum_norm || (c.no_pre_norm && !c.no_post_norm && c.norm_plain), FL_ERR_INVALID,
             "a norm of the sum is built for stacks whose sublayers read the stream itself, with plain norm weights");
    FL_CHECK(!(c.token_shift && c.canon_taps > 0), FL_ERR_UNSUPPORTED, "a stack has a token shift or input convolutions, not both");
    FL_CHECK(!c.token_shift || c.no_pre_norm, FL_ERR_UNSUPPORTED, "the token shift is built for stacks whose mixers read the stream itself");
    FL_CHECK(c.logit_softcap >= 0.f, FL_ERR_INVALID, "negative logit cap");
    m.W = c.width; m.V = c.vocab; m.L = c.n_layers; m.f32 = c.compute_dtype == FL_DTYPE_F32;
    m.layers.resize(m.L);
    struct Reg { void** pp; size_t bytes; };
    std::vector<Reg> regs;
    auto reg = [&](auto** pp, size_t bytes) { regs.push_back({(void**)pp, bytes}); };
    const size_t W = m.W;
    reg(&m.embed, (size_t)m.V * W * 2); reg(&m.head, (size_t)m.V * W * 2); reg(&m.final_norm, W * 4);
    if (c.max_positions > 0) reg(&m.pos, (size_t)c.max_positions * W * 2);
    auto pad8 = [](int n) { return (n + 7) / 8 * 8; };
    // one mixer: its rows inside the layer's stacked input matrix start at `base`; registers its side tables and its cache / state
    auto build_mixer = [&](LayeredLayerW& lw, int i, int base) {
        const fl_layer_desc& d = lw.d;
        const size_t H = d.heads, D = d.dim, Dv = d.vdim;
        auto recurrent = [&]() {                        // a per-slot state [heads][rows][vdim] + the per-head decay parameters
            lw.gla_index = (int)m.gla_layers.size();
            m.gla_layers.push_back(&lw);
            m.max_heads = std::max<int>(m.max_heads, (int)H);
        };
        auto rope = [&]() {
            const RopeSpec rs{d.rot_dims, d.rot_base, d.yarn_factor, d.yarn_original, d.yarn_fast, d.yarn_slow, d.rot_scaling};
            int ri = -1;
            for (size_t k = 0; k < m.ropes.size(); ++k)
                if (m.ropes[k] == rs) ri = (int)k;
            if (ri < 0) { ri = (int)m.ropes.size(); m.ropes.push_back(rs); }
            lw.rope_index = ri;
        };
        if (d.mixer == FL_MIXER_ATTN) {
            if (lw.d.kv_heads <= 0) lw.d.kv_heads = lw.d.heads;
            const size_t G = lw.d.kv_heads;
            lw.off_q = 0; lw.n_in = (int)(H * D); lw.off_k = lw.off_v = -1;
            if (!d.no_qk_norm) reg(&lw.qnorm, (d.qk_norm_whole ? H * D : D) * 4);
            if (d.qkv_bias) { reg(&lw.bq, H * D * 4); reg(&lw.bk, G * D * 4); reg(&lw.bv, G * Dv * 4); }
            if (d.sink == 2) reg(&lw.sinkv, H * 4);
            m.max_av = std::max<int>(m.max_av, (int)Dv);
            if (d.kv_from < 0) {
                lw.off_k = lw.n_in; lw.off_v = lw.off_k + (int)(G * D); lw.n_in = lw.off_v + (int)(G * Dv);
                if (!d.no_qk_norm) reg(&lw.knorm, (d.qk_norm_whole ? G * D : D) * 4);
                lw.kv_owner = i;
                lw.kv_index = (int)m.kv_layers.size();
                m.kv_layers.push_back(&lw);
            } else {
                lw.kv_owner = d.kv_from;
                lw.kv_index = m.layers[d.kv_from].kv_index;
            }
            lw.n_in = pad8(lw.n_in);
            rope();
        } else if (d.mixer == FL_MIXER_MAMBA2) {
            const size_t inner = H * Dv, GN = (size_t)d.groups * d.state;
            lw.off_g = 0;                               // z, the output gate
            lw.off_v = (int)inner; lw.off_k = (int)(2 * inner); lw.off_q = (int)(2 * inner + GN);    // x | B | C
            lw.off_dt = (int)(2 * inner + 2 * GN);
            lw.n_in = pad8(lw.off_dt + (int)H);
            lw.conv_off = (int)inner; lw.conv_ch = (int)(inner + 2 * GN);
            reg(&lw.conv_w, (size_t)lw.conv_ch * d.conv * 4); reg(&lw.conv_b, (size_t)lw.conv_ch * 4);
            reg(&lw.a_log, H * 4); reg(&lw.dt_bias, H * 4); reg(&lw.dskip, H * 4); reg(&lw.hnorm, inner * 4);
            recurrent();
        } else if (d.mixer == FL_MIXER_DELTA) {
            if (lw.d.kv_heads <= 0) lw.d.kv_heads = lw.d.heads;
            const size_t G = lw.d.kv_heads;
            lw.off_q = 0; lw.off_k = (int)(G * D); lw.off_v = (int)(2 * G * D); lw.off_g = lw.off_v + (int)(H * Dv);
            lw.off_b = lw.off_g + (int)(H * Dv); lw.off_a = lw.off_b + (int)H;
            lw.n_in = pad8(lw.off_a + (int)H);
            lw.conv_off = 0; lw.conv_ch = lw.off_g;
            reg(&lw.conv_w, (size_t)lw.conv_ch * d.conv * 4);
            reg(&lw.a_log, H * 4); reg(&lw.dt_bias, H * 4); reg(&lw.hnorm, Dv * 4);
            recurrent();
        } else if (d.mixer == FL_MIXER_LIGHTNING) {
            lw.off_q = 0; lw.off_k = (int)(H * D); lw.off_v = (int)(2 * H * D); lw.off_g = lw.off_v + (int)(H * Dv);
            lw.n_in = pad8(lw.off_g + (int)(H * Dv));
            lw.conv_off = 0; lw.conv_ch = lw.off_g;         // the activated span q | k | v (no convolution: conv = 0 taps)
            reg(&lw.decay, H * 4); reg(&lw.hnorm, H * Dv * 4);
            recurrent();
        } else if (d.mixer == FL_MIXER_GLA) {
            lw.off_q = 0; lw.off_k = (int)(H * D); lw.off_v = (int)(2 * H * D); lw.off_g = lw.off_v + (int)(H * Dv);
            lw.off_a = lw.off_g + (int)(H * Dv);
            lw.n_in = lw.off_a + d.decay_rank;
            reg(&lw.a2, H * D * d.decay_rank * 2); reg(&lw.a2b, H * D * 4); reg(&lw.hnorm, Dv * 4);
            lw.gla_index = (int)m.gla_layers.size();
            m.gla_layers.push_back(&lw);
            m.max_hd = std::max<int>(m.max_hd, (int)(H * D));
        } else {
            const size_t R = d.rot_dim, C = d.kv_rank;
            lw.off_q = 0; lw.n_in = (int)(H * (D + R));
            lw.off_dkv = -1;
            if (d.kv_from < 0) {
                lw.off_dkv = lw.n_in; lw.n_in += (int)(C + R);
                reg(&lw.dkv_norm, C * 4);
                lw.kv_owner = i;
                lw.kv_index = (int)m.kv_layers.size();
                m.kv_layers.push_back(&lw);
            } else {
                lw.kv_owner = d.kv_from;
                lw.kv_index = m.layers[d.kv_from].kv_index;
            }
            reg(&lw.uk_t, H * C * D * 2); reg(&lw.uv, H * Dv * C * 2);
            rope();
            m.max_hc = std::max<int>(m.max_hc, (int)(H * C));
        }
        if (base > 0) {             // rows of a second mixer: shift its offsets behind the first one's
            for (int* o : {&lw.off_q, &lw.off_k, &lw.off_v, &lw.off_g, &lw.off_a, &lw.off_dkv, &lw.off_b, &lw.off_dt})
                if (*o >= 0) *o += base;
            lw.conv_off += base;
        }
        reg(&lw.w_o, W * H * Dv * 2);
        m.max_hv = std::max<int>(m.max_hv, (int)(H * Dv));
        m.max_cv = std::max(m.max_cv, lw.conv_ch);
    };
    int next_desc = 0;
    for (int i = 0; i < m.L; ++i) {
        LayeredLayerW& lw = m.layers[i];
        lw.d = descs[next_desc++];
        const fl_layer_desc& d = lw.d;
        check_layer(m, i, d);
        const bool pre = !c.no_pre_norm, post = !c.no_post_norm;
        if (pre) reg(&lw.norm1, W * 4);
        if (post) reg(&lw.norm1b, W * 4);
        if (c.token_shift) reg(&lw.shift, W * 4);
        build_mixer(lw, i, 0);
        if (d.beside) {
            FL_CHECK(d.pair_sum ? c.post_sum_norm != 0 : !post, FL_ERR_UNSUPPORTED,
                     "mixers side by side: their normed mean joins the stream un-normed, or their weighted sum enters a norm of the sum");
            lw.side = std::make_shared<LayeredLayerW>();
            lw.side->d = descs[next_desc++];
            lw.side->d.beside = 0;
            check_mixer(m, i, lw.side->d, true);
            build_mixer(*lw.side, i, lw.n_in);
            lw.n_in += lw.side->n_in;
            lw.side->n_in = lw.n_in;                    // both read rows of the same projected buffer
            if (!d.pair_sum) { reg(&lw.pair_wa, W * 4); reg(&lw.pair_wb, W * 4); }
        }
        reg(&lw.w_in, (size_t)lw.n_in * W * 2);
        m.max_in = std::max(m.max_in, lw.n_in);
        if (c.canon_taps > 0) { reg(&lw.canon1, W * c.canon_taps * 4); lw.canon_index = i; }
        if (c.gated_residual) { reg(&lw.rg1, W * W * 2); reg(&lw.rg1b, W * 4); }
        if (c.depth_avg) reg(&lw.dwa, (size_t)(i + 2) * 4);
        if (d.ffn != FL_FFN_NONE) {
            if (pre) reg(&lw.norm2, W * 4);
            if (post) reg(&lw.norm2b, W * 4);
            if (c.canon_taps > 0) reg(&lw.canon2, W * c.canon_taps * 4);
            if (c.gated_residual) { reg(&lw.rg2, W * W * 2); reg(&lw.rg2b, W * 4); }
            if (d.ffn == FL_FFN_DENSE && d.ffn_bias) { reg(&lw.b_gu, (size_t)2 * d.ff * 4); reg(&lw.b_down, W * 4); }
            const size_t G = d.ffn == FL_FFN_MOE ? d.experts : 1, F = d.ff, GF = d.ffn_act == FL_ACT_RELU2 ? F : 2 * F;
            reg(&lw.w_gu, G * GF * W * 2); reg(&lw.w_down, G * W * F * 2);
            m.max_ff = std::max<int>(m.max_ff, (int)F);
            m.max_top = std::max(m.max_top, d.ffn == FL_FFN_MOE ? d.top : 1);
            if (d.ffn == FL_FFN_MOE) {
                reg(&lw.router, (size_t)d.experts * W * 4);
                if (d.router_bias) reg(&lw.router_b, (size_t)d.experts * 4);
                if (d.router == FL_ROUTER_SIGMOID_GROUPS) reg(&lw.route_corr, (size_t)d.experts * 4);
                m.max_experts = std::max(m.max_experts, d.experts);
                if (d.shared_ff > 0) {
                    reg(&lw.s_gu, (size_t)2 * d.shared_ff * W * 2); reg(&lw.s_down, W * (size_t)d.shared_ff * 2);
                    if (!d.shared_plain) reg(&lw.shared_gate, W * 4);
                    m.max_ff = std::max(m.max_ff, d.shared_ff);
                }
            }
        }
    }
    size_t total = 0;
    for (const Reg& r : regs) total += up256(r.bytes);
    m.slab.alloc(total, /*zero=*/true);
    size_t off = 0;
    for (const Reg& r : regs) { *r.pp = m.slab.p + off; off += up256(r.bytes); }
    m.weight_bytes = total - up256((size_t)m.V * W * 2) - (c.max_positions > 0 ? up256((size_t)c.max_positions * W * 2) : 0);

    // names -> destinations
    LayeredRoutes R;
    auto mat = [&](const std::string& n, uint16_t* base, int64_t row0, int64_t rows, int64_t cols) {
        R.r[n] = LyRoute{LyRoute::MAT16, base + row0 * cols, rows, cols, 0};
    };
    auto vec = [&](const std::string& n, float* base, int64_t rows, int64_t cols) { R.r[n] = LyRoute{LyRoute::F32, base, rows, cols, 0}; };
    // a layer norm's weight: [W], or one number for all channels (norm_scalar), kept as W equal floats so that the kernels index it alike
    auto normw = [&](const std::string& n, float* base) { R.r[n] = LyRoute{c.norm_scalar ? LyRoute::F32_FILL : LyRoute::F32, base, (int64_t)W, 1, 0}; };
    mat("embed", m.embed, 0, m.V, W); mat("head", m.head, 0, m.V, W); normw("final.norm", m.final_norm);
    if (m.pos != nullptr) mat("pos", m.pos, 0, c.max_positions, W);
    // the tensors of one mixer, named p + "q" and so on (p = "l<i>.mix." or "l<i>.mix.left." / "l<i>.mix.right.")
    auto route_mixer = [&](const LayeredLayerW& lw, const std::string& p) {
        const fl_layer_desc& d = lw.d;
        const int64_t H = d.heads, D = d.dim, Dv = d.vdim;
        if (d.mixer == FL_MIXER_ATTN) {
            const int64_t G = d.kv_heads;
            mat(p + "q", lw.w_in, lw.off_q, H * D, W);
            if (!d.no_qk_norm) vec(p + "q.norm", lw.qnorm, d.qk_norm_whole ? H * D : D, 1);
            if (d.kv_from < 0) {
                mat(p + "k", lw.w_in, lw.off_k, G * D, W); mat(p + "v", lw.w_in, lw.off_v, G * Dv, W);
                if (!d.no_qk_norm) vec(p + "k.norm", lw.knorm, d.qk_norm_whole ? G * D : D, 1);
            }
            if (d.qkv_bias) { vec(p + "q.b", lw.bq, H * D, 1); vec(p + "k.b", lw.bk, G * D, 1); vec(p + "v.b", lw.bv, G * Dv, 1); }
            if (d.sink == 2) vec(p + "sink", lw.sinkv, H, 1);
        } else if (d.mixer == FL_MIXER_MAMBA2) {
            mat(p + "in", lw.w_in, lw.off_g, lw.off_dt - lw.off_g + H, W);
            vec(p + "conv", lw.conv_w, lw.conv_ch, d.conv); vec(p + "conv.b", lw.conv_b, lw.conv_ch, 1);
            vec(p + "dt_bias", lw.dt_bias, H, 1); vec(p + "A_log", lw.a_log, H, 1); vec(p + "D", lw.dskip, H, 1);
            vec(p + "norm", lw.hnorm, H * Dv, 1);
        } else if (d.mixer == FL_MIXER_DELTA) {
            const int64_t G = d.kv_heads;
            mat(p + "q", lw.w_in, lw.off_q, G * D, W); mat(p + "k", lw.w_in, lw.off_k, G * D, W);
            mat(p + "v", lw.w_in, lw.off_v, H * Dv, W); mat(p + "g", lw.w_in, lw.off_g, H * Dv, W);
            mat(p + "b", lw.w_in, lw.off_b, H, W); mat(p + "a", lw.w_in, lw.off_a, H, W);
            vec(p + "q.conv", lw.conv_w + (size_t)(lw.off_q - lw.conv_off) * d.conv, G * D, d.conv);
            vec(p + "k.conv", lw.conv_w + (size_t)(lw.off_k - lw.conv_off) * d.conv, G * D, d.conv);
            vec(p + "v.conv", lw.conv_w + (size_t)(lw.off_v - lw.conv_off) * d.conv, H * Dv, d.conv);
            vec(p + "A_log", lw.a_log, H, 1); vec(p + "dt_bias", lw.dt_bias, H, 1); vec(p + "norm", lw.hnorm, Dv, 1);
        } else if (d.mixer == FL_MIXER_LIGHTNING) {
            mat(p + "q", lw.w_in, lw.off_q, H * D, W); mat(p + "k", lw.w_in, lw.off_k, H * D, W);
            mat(p + "v", lw.w_in, lw.off_v, H * Dv, W); mat(p + "g", lw.w_in, lw.off_g, H * Dv, W);
            vec(p + "norm", lw.hnorm, H * Dv, 1);
            R.r[p + "decay"] = LyRoute{LyRoute::F32_RAW, lw.decay, H, 1, 0};
        } else if (d.mixer == FL_MIXER_GLA) {
            mat(p + "q", lw.w_in, lw.off_q, H * D, W); mat(p + "k", lw.w_in, lw.off_k, H * D, W);
            mat(p + "v", lw.w_in, lw.off_v, H * Dv, W); mat(p + "g", lw.w_in, lw.off_g, H * Dv, W);
            mat(p + "a1", lw.w_in, lw.off_a, d.decay_rank, W);
            mat(p + "a2", lw.a2, 0, H * D, d.decay_rank); vec(p + "a2.b", lw.a2b, H * D, 1); vec(p + "norm", lw.hnorm, Dv, 1);
        } else {
            const int64_t Rr = d.rot_dim, C = d.kv_rank;
            mat(p + "q", lw.w_in, lw.off_q, H * (D + Rr), W);
            if (d.kv_from < 0) { mat(p + "dkv", lw.w_in, lw.off_dkv, C + Rr, W); vec(p + "dkv.norm", lw.dkv_norm, C, 1); }
            R.r[p + "uk"] = LyRoute{LyRoute::UK_T, lw.uk_t, H * D, C, (int)H};
            mat(p + "uv", lw.uv, 0, H * Dv, C);
        }
        mat(p + "o", lw.w_o, 0, W, H * Dv);
    };
    for (int i = 0; i < m.L; ++i) {
        LayeredLayerW& lw = m.layers[i];
        const fl_layer_desc& d = lw.d;
        const std::string p = "l" + std::to_string(i) + ".";
        const bool pre = !c.no_pre_norm, post = !c.no_post_norm;
        if (pre && post) { normw(p + "norm1", lw.norm1); normw(p + "norm1b", lw.norm1b); }
        else normw(p + "norm1", pre ? lw.norm1 : lw.norm1b);
        if (lw.shift) vec(p + "shift", lw.shift, W, 1);
        if (lw.side) {
            lw.side->w_in = lw.w_in;
            route_mixer(lw, p + "mix.left."); route_mixer(*lw.side, p + "mix.right.");
            if (lw.pair_wa) { vec(p + "mix.left.out", lw.pair_wa, W, 1); vec(p + "mix.right.out", lw.pair_wb, W, 1); }
        } else {
            route_mixer(lw, p + "mix.");
        }
        if (lw.canon1) vec(p + "canon1", lw.canon1, W, c.canon_taps);
        if (lw.rg1) { mat(p + "rg1", lw.rg1, 0, W, W); vec(p + "rg1.b", lw.rg1b, W, 1); }
        if (lw.dwa) vec(p + "dwa", lw.dwa, i + 2, 1);
        if (d.ffn == FL_FFN_NONE) continue;
        if (pre && post) { normw(p + "norm2", lw.norm2); normw(p + "norm2b", lw.norm2b); }
        else normw(p + "norm2", pre ? lw.norm2 : lw.norm2b);
        if (lw.canon2) vec(p + "canon2", lw.canon2, W, c.canon_taps);
        if (lw.rg2) { mat(p + "rg2", lw.rg2, 0, W, W); vec(p + "rg2.b", lw.rg2b, W, 1); }
        const int64_t F = d.ff;
        const bool gated = d.ffn_act != FL_ACT_RELU2;
        const int64_t GF = gated ? 2 * F : F;
        if (d.ffn == FL_FFN_DENSE) {
            if (gated) mat(p + "mlp.gate", lw.w_gu, 0, F, W);
            mat(p + "mlp.up", lw.w_gu, gated ? F : 0, F, W); mat(p + "mlp.down", lw.w_down, 0, W, F);
            if (d.ffn_bias) {
                vec(p + "mlp.gate.b", lw.b_gu, F, 1); vec(p + "mlp.up.b", lw.b_gu + F, F, 1); vec(p + "mlp.down.b", lw.b_down, W, 1);
            }
        } else {
            vec(p + "mlp.router", lw.router, d.experts, W);
            if (lw.router_b) vec(p + "mlp.router.b", lw.router_b, d.experts, 1);
            if (lw.route_corr) vec(p + "mlp.correction", lw.route_corr, d.experts, 1);
            for (int e = 0; e < d.experts; ++e) {
                const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                if (gated) mat(q + "gate", lw.w_gu, (int64_t)e * GF, F, W);
                mat(q + "up", lw.w_gu, (int64_t)e * GF + (gated ? F : 0), F, W);
                mat(q + "down", lw.w_down, (int64_t)e * W, W, F);
            }
            if (d.shared_ff > 0) {
                const int64_t Fs = d.shared_ff;
                mat(p + "mlp.shared.gate", lw.s_gu, 0, Fs, W); mat(p + "mlp.shared.up", lw.s_gu, Fs, Fs, W);
                mat(p + "mlp.shared.down", lw.s_down, 0, W, Fs);
                if (lw.shared_gate) vec(p + "mlp.shared.sg", lw.shared_gate, 1, W);
            }
        }
    }
    for (const auto& kv : R.r) m.expected.push_back(kv.first);
    std::lock_guard<std::mutex> g(g_routes_mu);
    g_routes[&m] = std::move(R);
}

static const LyRoute* find_route(const LayeredModel& m, const std::string& name) {
    std::lock_guard<std::mutex> g(g_routes_mu);
    auto it = g_routes.find(&m);
    if (it == g_routes.end()) return nullptr;
    auto jt = it->second.r.find(name);
    return jt == it->second.r.end() ? nullptr : &jt->second;
}

void layered_put_tensor(LayeredModel& m, const char* name, int dtype, const int64_t* shape, int rank, const void* host) {
    FL_CHECK(!m.finalized, FL_ERR_STATE, "model already finalized");
    const LyRoute* r = find_route(m, name);
    if (r == nullptr) { m.ignored++; return; }       // a tensor the layers do not read
    int64_t numel = 1;
    for (int i = 0; i < rank; ++i) numel *= shape[i];
    const bool shape_ok = r->kind == LyRoute::F32_FILL
                              ? numel == 1
                              : numel == r->rows * r->cols && (rank == 1 || (rank == 2 && (shape[0] == r->rows || r->cols == 1 || r->rows == 1)));
    FL_CHECK(shape_ok, FL_ERR_INVALID, std::string("shape mismatch for ") + name);
    FL_CHECK(dtype == FL_DTYPE_F32 || dtype == FL_DTYPE_BF16 || dtype == FL_DTYPE_F16, FL_ERR_INVALID, "bad dtype");
    if (r->kind == LyRoute::F32_RAW && dtype == FL_DTYPE_F32) {
        FL_CUDA(cudaMemcpy(r->dst, host, (size_t)numel * 4, cudaMemcpyHostToDevice));
        m.have.insert(name);
        return;
    }
    std::vector<uint16_t> bits((size_t)numel);
    if (dtype == FL_DTYPE_BF16) std::memcpy(bits.data(), host, (size_t)numel * 2);
    else if (dtype == FL_DTYPE_F32) for (int64_t i = 0; i < numel; ++i) bits[i] = f32_to_bits(((const float*)host)[i]);
    else for (int64_t i = 0; i < numel; ++i) bits[i] = f32_to_bits(half_to_f32(((const uint16_t*)host)[i]));
    if (r->kind == LyRoute::MAT16) {
        FL_CUDA(cudaMemcpy(r->dst, bits.data(), (size_t)numel * 2, cudaMemcpyHostToDevice));
    } else if (r->kind == LyRoute::F32 || r->kind == LyRoute::F32_RAW) {
        std::vector<float> v((size_t)numel);
        for (int64_t i = 0; i < numel; ++i) v[i] = bits_to_f32(bits[i]);
        FL_CUDA(cudaMemcpy(r->dst, v.data(), (size_t)numel * 4, cudaMemcpyHostToDevice));
    } else if (r->kind == LyRoute::F32_FILL) {
        std::vector<float> v((size_t)(r->rows * r->cols), bits_to_f32(bits[0]));
        FL_CUDA(cudaMemcpy(r->dst, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
    } else {        // [heads * D, C] -> [heads][C][D]
        const int64_t Hh = r->heads, D = r->rows / Hh, C = r->cols;
        std::vector<uint16_t> t((size_t)numel);
        for (int64_t h = 0; h < Hh; ++h)
            for (int64_t d = 0; d < D; ++d)
                for (int64_t c = 0; c < C; ++c) t[(size_t)((h * C + c) * D + d)] = bits[(size_t)((h * D + d) * C + c)];
        FL_CUDA(cudaMemcpy(r->dst, t.data(), (size_t)numel * 2, cudaMemcpyHostToDevice));
    }
    m.have.insert(name);
}

void layered_random_init(LayeredModel& m, uint64_t seed, float stdv) {
    FL_CHECK(!m.finalized, FL_ERR_STATE, "model already finalized");
    const RowMap ident{0, 0, 0, 0};
    for (const std::string& n : m.expected) {
        const LyRoute* r = find_route(m, n);
        const uint64_t ts = tensor_seed(seed, n.c_str());
        const int64_t numel = r->rows * r->cols;
        if (r->kind == LyRoute::F32 || r->kind == LyRoute::F32_RAW || r->kind == LyRoute::F32_FILL) {
            auto ends = [&](const char* t) { const size_t k = std::strlen(t); return n.size() >= k && n.compare(n.size() - k, k, t) == 0; };
            // a plain norm weight sits around one, a zero-centred one around zero
            const bool around_one = ends("mix.norm") || ends("left.norm") || ends("right.norm") || ends("dkv.norm") || ends("q.norm") || ends("k.norm") || ends("mix.D") || ends("left.out") || ends("right.out") ||
                                    (m.cfg.norm_plain && (ends("norm1") || ends("norm2") || ends("norm1b") || ends("norm2b") || n == "final.norm"));
            const bool is_mat = n.find("router") != std::string::npos || n.find("mix.a2") != std::string::npos || n.find("shared.sg") != std::string::npos ||
                                ends(".conv") || ends(".canon1") || ends(".canon2");
            const bool is_bias = n.size() >= 4 && n.compare(n.size() - 4, 4, "a2.b") == 0;
            if (around_one) fill_f32_kernel<<<8, 256>>>((float*)r->dst, numel, 1.0f);
            else if (ends(".decay")) fill_f32_kernel<<<8, 256>>>((float*)r->dst, numel, 0.96875f);
            else if (ends(".shift")) fill_f32_kernel<<<8, 256>>>((float*)r->dst, numel, 0.25f);
            else if (ends(".dwa")) fill_f32_kernel<<<8, 256>>>((float*)r->dst, numel, 1.0f / (float)numel);     // a plain mean over the outputs so far
            else if (is_bias) fill_f32_kernel<<<8, 256>>>((float*)r->dst, numel, 3.0f);
            else if (is_mat) synth_fill_f32_kernel<<<kNumSMs, 256>>>((float*)r->dst, numel, ts, stdv, ident);
            else fill_f32_kernel<<<8, 256>>>((float*)r->dst, numel, 0.0f);
        } else {
            synth_fill_bf16_kernel<<<kNumSMs * 8, 256>>>((uint16_t*)r->dst, 1, numel, numel, ts, n == "embed" ? 1.0f : stdv, ident);
        }
        g_launches.fetch_add(1);
        m.have.insert(n);
    }
    FL_CUDA(cudaGetLastError());
    FL_CUDA(cudaDeviceSynchronize());
}

void layered_finalize(LayeredModel& m) {
    FL_CHECK(!m.finalized, FL_ERR_STATE, "model already finalized");
    for (const std::string& n : m.expected) FL_CHECK(m.have.count(n), FL_ERR_STATE, "missing tensor: " + n);
    {
        std::lock_guard<std::mutex> g(g_routes_mu);
        g_routes.erase(&m);
    }
    // serving precision: the projections whose shapes fit the tcgen05 GEMM's tiles (whole 64-column k blocks, 16-byte rows) run
    // there; everything else, and every product of the exact mode, stays on the f32 FMA kernel
    if (!m.f32 && !env_flag("FL_LAYERED_NO_TC")) {
        auto fits = [](int N, int K) { return K % 64 == 0 && N % 8 == 0; };
        auto map = [&](const uint16_t* p, int N, int K, CUtensorMap& tm, bool& ok) {
            ok = p != nullptr && fits(N, K);
            if (ok) tm = make_tmap_bf16(p, (uint64_t)N, (uint64_t)K, (uint64_t)K, 128);
        };
        for (LayeredLayerW& lw : m.layers) {
            const fl_layer_desc& d = lw.d;
            map(lw.w_in, lw.n_in, m.W, lw.tm_in, lw.tc_in);
            map(lw.w_o, m.W, d.heads * d.vdim, lw.tm_o, lw.tc_o);
            if (lw.side) map(lw.side->w_o, m.W, lw.side->d.heads * lw.side->d.vdim, lw.side->tm_o, lw.side->tc_o);
            map(lw.rg1, m.W, m.W, lw.tm_rg1, lw.tc_rg1); map(lw.rg2, m.W, m.W, lw.tm_rg2, lw.tc_rg2);
            const int GF = d.ffn_act == FL_ACT_RELU2 ? d.ff : 2 * d.ff;       // rows of the first feed-forward matrix: up, or gate | up
            if (d.ffn == FL_FFN_DENSE) { map(lw.w_gu, GF, m.W, lw.tm_gu, lw.tc_gu); map(lw.w_down, m.W, d.ff, lw.tm_down, lw.tc_down); }
            if (d.ffn == FL_FFN_MOE && d.shared_ff > 0) {
                map(lw.s_gu, 2 * d.shared_ff, m.W, lw.tm_sgu, lw.tc_sgu); map(lw.s_down, m.W, d.shared_ff, lw.tm_sdown, lw.tc_sdown);
            }
            if (d.ffn == FL_FFN_MOE && fits(GF, m.W) && fits(m.W, d.ff)) {
                lw.tc_moe = true;
                lw.tm_gu = make_tmap_bf16(lw.w_gu, (uint64_t)d.experts * GF, (uint64_t)m.W, (uint64_t)m.W, 128);
                lw.tm_down = make_tmap_bf16(lw.w_down, (uint64_t)d.experts * m.W, (uint64_t)d.ff, (uint64_t)d.ff, 128);
                for (int e = 0; e < d.experts; ++e) {
                    lw.tm_egu.push_back(make_tmap_bf16(lw.w_gu + (size_t)e * GF * m.W, (uint64_t)GF, (uint64_t)m.W, (uint64_t)m.W, 128));
                    lw.tm_edown.push_back(make_tmap_bf16(lw.w_down + (size_t)e * m.W * d.ff, (uint64_t)m.W, (uint64_t)d.ff, (uint64_t)d.ff, 128));
                }
            }
        }
        map(m.head, m.V, m.W, m.tm_head, m.tc_head);
    }
    // the norm of the sum parks a row in shared memory: above the default 48 KB the kernels are told so once
    if (m.cfg.post_sum_norm && (size_t)m.W * 4 > 48 * 1024) {
        FL_CHECK((size_t)m.W * 4 <= 200 * 1024, FL_ERR_UNSUPPORTED, "a norm of the sum is built for widths up to 51200");
        FL_CUDA(cudaFuncSetAttribute(ly_sum_norm_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, m.W * 4));
        FL_CUDA(cudaFuncSetAttribute(ly_sum_norm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, m.W * 4));
    }
    m.finalized = true;
}

// ---- cache -------------------------------------------------------------------------------------------------------------------
static void rope_tables(const RopeSpec& rs, int max_seq, std::vector<float>& cs, std::vector<float>& sn) {
    const int half = rs.dims / 2;
    std::vector<double> f(half);
    double mult = 1.0;
    for (int i = 0; i < half; ++i) f[i] = std::pow(rs.base, -2.0 * i / (double)rs.dims);
    if (rs.yarn_factor > 0.f && rs.scaling == FL_ROT_SCALE_BANDS) {
        // bands of wavelength: short ones (below original / fast) keep their frequency, long ones (above original / slow) are slowed
        // by the factor, between the two a linear blend in original / wavelength; magnitude 1
        const double factor = rs.yarn_factor, orig = rs.yarn_original, hi = rs.yarn_fast, lo = rs.yarn_slow;
        for (int i = 0; i < half; ++i) {
            const double wl = 2.0 * M_PI / f[i];
            if (wl < orig / hi) continue;
            if (wl > orig / lo) { f[i] /= factor; continue; }
            const double sm = (orig / wl - lo) / (hi - lo);
            f[i] = (1.0 - sm) * f[i] / factor + sm * f[i];
        }
    } else if (rs.yarn_factor > 0.f) {
        // YaRN: pairs that complete many turns inside the original context keep their frequency, slow pairs are stretched by the
        // factor, a linear ramp between the two pair indices; cos and sin grow by 0.1 ln(factor) + 1
        const double factor = rs.yarn_factor, orig = rs.yarn_original;
        auto corr = [&](double turns) { return rs.dims * std::log(orig / (2.0 * M_PI * turns)) / (2.0 * std::log(rs.base)); };
        const double lo = std::max(std::floor(corr(rs.yarn_fast)), 0.0), hi = std::min(std::ceil(corr(rs.yarn_slow)), (double)rs.dims - 1.0);
        for (int i = 0; i < half; ++i) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp);
        }
        mult = 0.1 * std::log(factor) + 1.0;
    }
    cs.resize((size_t)max_seq * half); sn.resize((size_t)max_seq * half);
    for (int p = 0; p < max_seq; ++p)
        for (int i = 0; i < half; ++i) {
            cs[(size_t)p * half + i] = (float)(std::cos(p * f[i]) * mult);
            sn[(size_t)p * half + i] = (float)(std::sin(p * f[i]) * mult);
        }
}

void layered_cache_create(fl_cache& c, int max_slots, int max_seq, int pool_tokens) {
    const LayeredModel& m = *c.lm;
    FL_CHECK(m.finalized, FL_ERR_STATE, "model not finalized");
    FL_CHECK(max_slots >= 1 && max_slots <= kMaxBatch && max_seq >= 1 && pool_tokens >= 1, FL_ERR_INVALID, "bad cache dimensions");
    c.max_batch = max_slots; c.max_seq = max_seq;
    c.pages_per_seq = (max_seq + kKvPage - 1) / kKvPage;
    FL_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    c.ly.reset(new LayeredCache);
    LayeredCache& y = *c.ly;
    y.f32 = m.f32;
    const int pages = (pool_tokens + kKvPage - 1) / kKvPage;
    y.pool = PagePool(pages, max_slots, c.pages_per_seq, kKvPage);
    const size_t esz = m.f32 ? 4 : 2;
    y.kv_store.resize(m.kv_layers.size());
    for (size_t k = 0; k < m.kv_layers.size(); ++k) {
        const fl_layer_desc& d = m.kv_layers[k]->d;
        const size_t width = d.mixer == FL_MIXER_ATTN ? (size_t)d.kv_heads * (d.dim + d.vdim) : (size_t)(d.kv_rank + d.rot_dim);
        y.kv_store[k].alloc((size_t)pages * kKvPage * width * esz, true);
        y.kv_pool.push_back(y.kv_store[k].p);
    }
    y.gla_state.resize(m.gla_layers.size());
    y.conv_state.resize(m.gla_layers.size());
    for (size_t k = 0; k < m.gla_layers.size(); ++k) {
        const LayeredLayerW& lw = *m.gla_layers[k];
        const fl_layer_desc& d = lw.d;
        const size_t rows = d.mixer == FL_MIXER_MAMBA2 ? d.state : d.dim;
        y.gla_state[k].alloc((size_t)max_slots * d.heads * rows * d.vdim, true);
        if (lw.conv_ch > 0 && d.conv > 1) y.conv_state[k].alloc((size_t)max_slots * (d.conv - 1) * lw.conv_ch, true);
    }
    if (m.cfg.canon_taps > 1) {
        y.canon_state.resize(m.L);
        for (int i = 0; i < m.L; ++i) y.canon_state[i].alloc((size_t)2 * max_slots * (m.cfg.canon_taps - 1) * m.W, true);
    }
    if (m.cfg.token_shift) {
        y.shift_state.resize(m.L);
        for (int i = 0; i < m.L; ++i) y.shift_state[i].alloc((size_t)max_slots * m.W, true);
    }
    y.rope_cos.resize(m.ropes.size()); y.rope_sin.resize(m.ropes.size());
    for (size_t k = 0; k < m.ropes.size(); ++k) {
        std::vector<float> cs, sn;
        rope_tables(m.ropes[k], max_seq, cs, sn);
        y.rope_cos[k].alloc(std::max<size_t>(cs.size(), 1)); y.rope_sin[k].alloc(std::max<size_t>(sn.size(), 1));
        if (!cs.empty()) {
            FL_CUDA(cudaMemcpy(y.rope_cos[k].p, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
            FL_CUDA(cudaMemcpy(y.rope_sin[k].p, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
        }
    }
    y.page_table.alloc((size_t)max_slots * c.pages_per_seq, true);
    if (m.max_av > 0 && !m.f32) y.at_part.alloc((size_t)kGqaSplitRows * kGqaMaxSplits * (m.max_av + 2));
    c.slot_len.assign(max_slots, 0);
    FL_CUDA(cudaDeviceSynchronize());
}

void layered_slot_reset(fl_cache& c, int slot) {
    c.ly->pool.release(slot);       // the recurrent state needs no clearing: a sequence that starts at position 0 starts from zero
    c.slot_len[slot] = 0;
}

void layered_cache_reset(fl_cache& c) {
    for (int s = 0; s < c.max_batch; ++s) layered_slot_reset(c, s);
}

// captured decode steps hold workspace pointers: they go when a buffer they name is reallocated
static void drop_graphs(fl_cache& c) {
    for (auto& kv : c.graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    c.graphs.clear();
}

static void ensure_ws(fl_cache& c, size_t T, size_t n_want) {
    const LayeredModel& m = *c.lm;
    LayeredCache& y = *c.ly;
    if (T > y.rows) {
        FL_CUDA(cudaStreamSynchronize(c.stream));
        drop_graphs(c);
        const size_t R = std::max<size_t>(T, 2 * y.rows), W = m.W, P = R * std::max(m.max_top, 1);
        y.x.alloc(R * W); y.h.alloc(R * W); y.y.alloc(R * W);
        y.proj.alloc(R * m.max_in); y.u.alloc(R * std::max(m.max_hv, 1)); y.go.alloc(R * std::max(m.max_hv, 1));
        y.la.alloc(R * std::max(m.max_hd, 1));
        y.cv.alloc(R * std::max(m.max_cv, 1)); y.rs.alloc(R * 2 * std::max(m.max_heads, 1));
        if (m.cfg.canon_taps > 0 || m.cfg.token_shift) y.hc.alloc(R * W);
        if (m.cfg.gated_residual) y.gz.alloc(R * W);
        if (m.cfg.depth_avg) y.xs.alloc((size_t)(m.L + 1) * R * W);
        for (const LayeredLayerW& lw : m.layers)
            if (lw.side && y.y2.n < R * W) y.y2.alloc(R * W);
        y.qa.alloc(R * std::max(m.max_hc, 1)); y.ol.alloc(R * std::max(m.max_hc, 1));
        y.gu.alloc(P * 2 * std::max(m.max_ff, 1)); y.act.alloc(P * std::max(m.max_ff, 1)); y.eo.alloc(P * W);
        y.sh_gu.alloc(R * 2 * std::max(m.max_ff, 1)); y.sh_act.alloc(R * std::max(m.max_ff, 1)); y.sh_o.alloc(R * W);
        y.route_w.alloc(P); y.route_sel.alloc(P); y.sgate.alloc(R);
        y.pair_row.alloc(P); y.pair_of.alloc(P); y.grp_off.alloc((size_t)m.max_experts + 2);
        if (!m.f32) {
            y.h_hi.alloc(R * W); y.h_lo.alloc(R * W);
            y.u_hi.alloc(R * std::max(m.max_hv, 1)); y.u_lo.alloc(R * std::max(m.max_hv, 1));
            y.act_hi.alloc(R * std::max(m.max_ff, 1)); y.act_lo.alloc(R * std::max(m.max_ff, 1));
            // split-K slices of a tensor-core GEMM with <= 128 rows: ks * rows <= 256 (see pick_ksplit)
            const size_t nmax = std::max<size_t>(std::max<size_t>(m.max_in, W), std::max<size_t>(2 * (size_t)m.max_ff, m.V));
            size_t need = 256 * nmax;
            size_t gx_rows = 0;
            for (const LayeredLayerW& lw : m.layers) {          // grouped expert GEMMs: [slices][experts * cap rows][2 ff | W]
                if (!lw.tc_moe) continue;
                const int E = lw.d.experts, F = lw.d.ff, GF = lw.d.ffn_act == FL_ACT_RELU2 ? F : 2 * F;
                gx_rows = std::max<size_t>(gx_rows, (size_t)E * 128);
                for (int cap = 16; cap <= 128; cap *= 2) {
                    const int k1 = pick_ksplit(E * ((GF + 127) / 128), (int)(W + 63) / 64, cap), k2 = pick_ksplit(E * ((int)(W + 127) / 128), (F + 63) / 64, cap);
                    need = std::max(need, std::max((size_t)k1 * E * cap * GF, (size_t)k2 * E * cap * W));
                }
            }
            if (y.gemm_out.n < need) y.gemm_out.alloc(need);
            if (gx_rows > 0 && y.gx_hi.n == 0) {
                y.gx_hi.alloc(gx_rows * W, true); y.gx_lo.alloc(gx_rows * W, true);
                y.ga_hi.alloc(gx_rows * std::max(m.max_ff, 1), true); y.ga_lo.alloc(gx_rows * std::max(m.max_ff, 1), true);
                y.grp_cnt.alloc((size_t)m.max_experts + 1, true);
            }
        }
        y.rows = R;
    }
    if (n_want > y.want_cap) {
        FL_CUDA(cudaStreamSynchronize(c.stream));
        drop_graphs(c);
        const size_t N = std::max<size_t>(n_want, 2 * y.want_cap);
        y.hf.alloc(N * m.W); y.logits.alloc(N * m.V); y.h_logits.alloc(N * m.V);
        if (!m.f32) { y.hf_hi.alloc(N * m.W); y.hf_lo.alloc(N * m.W); }
        y.want_cap = N;
    }
}

// The FMA-chain GEMM: f32 accumulators where it stands in for the tensor-core GEMM on shapes outside its tiles (serving precision),
// f64 accumulators in the exact mode.
static void gemm(LaunchCtx& lc, const char* tag, const float* A, int lda, const uint16_t* Wt, int N, int K, float* Y, int ldy, int R) {
    if (R <= 0) return;
    LyGemm g{A, 0, lda, nullptr, Wt, 0, N, K, Y, 0, ldy, nullptr, R};
    const dim3 grid((N + kLyBN - 1) / kLyBN, (R + kLyBM - 1) / kLyBM, 1);
    if (lc.exact) launch(lc, tag, (uint64_t)N * K * 2, ly_gemm_kernel<double>, grid, dim3(256), 0, g);
    else launch(lc, tag, (uint64_t)N * K * 2, ly_gemm_kernel<float>, grid, dim3(256), 0, g);
}
// Y[R, N] = A[R, K] . Wt[N, K]^T on the tensor cores when the matrix has a descriptor (serving precision; A as hi | lo halves),
// else on the exact kernel.  Split-K slices of the tensor-core GEMM are folded in slice order.
static void gemm_tc_or_exact(fl_cache& c, LaunchCtx& lc, const char* tag, const float* A, const uint16_t* ahi, const uint16_t* alo, const uint16_t* Wt,
                             const CUtensorMap& tm, bool tc, int N, int K, float* Y, int R) {
    if (R <= 0) return;
    if (!tc || ahi == nullptr) { gemm(lc, tag, A, K, Wt, N, K, Y, N, R); return; }
    LayeredCache& y = *c.ly;
    const int ks_plan = R <= 128 ? pick_ksplit((N + 127) / 128, (K + 63) / 64, R) : 1;
    float* out = ks_plan == 1 ? Y : y.gemm_out.p;
    FL_CHECK(ks_plan == 1 || (size_t)ks_plan * R * N <= y.gemm_out.n, FL_ERR_STATE, "internal: split-K scratch too small");
    const int ks = dense_gemm(c, lc, tag, R, N, K, tm, out, ahi, alo);
    FL_CHECK(ks == ks_plan, FL_ERR_STATE, "internal: split-K plan mismatch");
    if (ks > 1) {
        const size_t n = (size_t)R * N;
        launch(lc, "sum_slices", 0, ly_sum_slices_kernel, dim3((unsigned)std::min<size_t>(4 * kNumSMs, (n + 255) / 256)), dim3(256), 0,
               (const float*)out, ks, n, n, Y);
    }
}

static void gemm_groups(LaunchCtx& lc, const char* tag, const LyGemm& g, int groups, int max_rows) {
    if (max_rows <= 0) return;
    const dim3 grid((g.N + kLyBN - 1) / kLyBN, (max_rows + kLyBM - 1) / kLyBM, groups);
    if (lc.exact) launch(lc, tag, (uint64_t)groups * g.N * g.K * 2, ly_gemm_kernel<double>, grid, dim3(256), 0, g);
    else launch(lc, tag, (uint64_t)groups * g.N * g.K * 2, ly_gemm_kernel<float>, grid, dim3(256), 0, g);
}

template <typename CT>
static void launch_latent_attn(LaunchCtx& lc, const LatentAttnArgs& a, int T) {
    const int cpl = (a.C + 31) / 32;
    const size_t smem = ((size_t)kLatWarps * a.C + 2 * kLatWarps) * 4;
    const dim3 g(T, a.H), b(kLatWarps * 32);
    const uint64_t bytes = 0;
    if (cpl <= 1) launch(lc, "latent_attn", bytes, ly_latent_attn_kernel<CT, 1>, g, b, smem, a);
    else if (cpl <= 2) launch(lc, "latent_attn", bytes, ly_latent_attn_kernel<CT, 2>, g, b, smem, a);
    else if (cpl <= 4) launch(lc, "latent_attn", bytes, ly_latent_attn_kernel<CT, 4>, g, b, smem, a);
    else if (cpl <= 8) launch(lc, "latent_attn", bytes, ly_latent_attn_kernel<CT, 8>, g, b, smem, a);
    else launch(lc, "latent_attn", bytes, ly_latent_attn_kernel<CT, 16>, g, b, smem, a);
}

static void launch_gla_scan(LaunchCtx& lc, const GlaArgs& a, int n) {
    const int rpt = (a.D + kGlaDG - 1) / kGlaDG;
    const size_t smem = ((size_t)6 * a.D + 2 * kGlaVS + 2 * kGlaDG * kGlaVS) * 4;
    const dim3 g(n, a.H, (a.Dv + kGlaVS - 1) / kGlaVS), b(kGlaVS * kGlaDG);
    if (rpt <= 1) launch(lc, "gla_scan", 0, ly_gla_scan_kernel<1>, g, b, smem, a);
    else if (rpt <= 2) launch(lc, "gla_scan", 0, ly_gla_scan_kernel<2>, g, b, smem, a);
    else if (rpt <= 4) launch(lc, "gla_scan", 0, ly_gla_scan_kernel<4>, g, b, smem, a);
    else if (rpt <= 8) launch(lc, "gla_scan", 0, ly_gla_scan_kernel<8>, g, b, smem, a);
    else if (rpt <= 16) launch(lc, "gla_scan", 0, ly_gla_scan_kernel<16>, g, b, smem, a);
    else launch(lc, "gla_scan", 0, ly_gla_scan_kernel<32>, g, b, smem, a);
}

template <typename CT, int RB>
static void launch_gqa_attn_rb(LaunchCtx& lc, const GqaAttnArgs& a, int T, int splits) {
    const int cpl = (std::max(a.D, a.Dv) + 31) / 32;
    const size_t smem = ((size_t)kGqaWarps * RB * (a.Dv + 2)) * 4;
    const dim3 g(T, a.H / RB, splits), b(kGqaWarps * 32);
    if (cpl <= 1) launch(lc, "gqa_attn", 0, ly_gqa_attn_kernel<CT, 1, RB>, g, b, smem, a);
    else if (cpl <= 2) launch(lc, "gqa_attn", 0, ly_gqa_attn_kernel<CT, 2, RB>, g, b, smem, a);
    else if (cpl <= 4) launch(lc, "gqa_attn", 0, ly_gqa_attn_kernel<CT, 4, RB>, g, b, smem, a);
    else launch(lc, "gqa_attn", 0, ly_gqa_attn_kernel<CT, 8, RB>, g, b, smem, a);
}
// max_keys: the most keys a row of the launch can see (bounds the useful number of key splits).  The exact mode never splits: there
// a position's result is bitwise the same whatever else the launch holds.
template <typename CT>
static void launch_gqa_attn(LaunchCtx& lc, const GqaAttnArgs& a, int T, int max_keys, bool may_split) {
    if (T <= 0) return;
    const int rep = a.H / a.G, rb = rep % 4 == 0 ? 4 : (rep % 2 == 0 ? 2 : 1);
    int splits = 1;
    if (may_split && a.part != nullptr && (long long)T * a.H <= kGqaSplitRows) {
        const int blocks = T * (a.H / rb);
        splits = std::min(kGqaMaxSplits, std::max(1, 2 * kNumSMs / std::max(blocks, 1)));
        splits = std::max(1, std::min(splits, max_keys / (kGqaWarps * 16)));        // at least 16 keys per warp
    }
    if (rb == 4) launch_gqa_attn_rb<CT, 4>(lc, a, T, splits);
    else if (rb == 2) launch_gqa_attn_rb<CT, 2>(lc, a, T, splits);
    else launch_gqa_attn_rb<CT, 1>(lc, a, T, splits);
    if (splits > 1)
        launch(lc, "gqa_merge", 0, ly_gqa_merge_kernel, dim3(T, a.H), dim3(std::min(256, std::max(32, (a.Dv + 31) / 32 * 32))), 0, (const float*)a.part, splits,
               a.H, a.Dv, a.sink, a.sinkv, a.row_base, a.out, a.ohi, a.olo);
}

template <bool DELTA>
static void launch_rec_scan(LaunchCtx& lc, const RecArgs& a, int n) {
    const int rpt = (a.D + kRecParts - 1) / kRecParts;
    auto go = [&](auto kern, int RPT) {
        const size_t smem = (size_t)4 * (RPT >= 64 ? 4 : 8) * (2 * kRecParts * (RPT + 4) + 12) * 4;       // [4 warps][ring][slot] floats
        launch(lc, DELTA ? "delta_scan" : "ssm_scan", 0, kern, dim3(n, a.H, (a.Dv + kRecCols - 1) / kRecCols), dim3(128), smem, a);
    };
    if (rpt <= 2) go(ly_rec_scan_kernel<2, DELTA>, 2);
    else if (rpt <= 4) go(ly_rec_scan_kernel<4, DELTA>, 4);
    else if (rpt <= 8) go(ly_rec_scan_kernel<8, DELTA>, 8);
    else if (rpt <= 16) go(ly_rec_scan_kernel<16, DELTA>, 16);
    else if (rpt <= 32) go(ly_rec_scan_kernel<32, DELTA>, 32);
    else go(ly_rec_scan_kernel<64, DELTA>, 64);
}

// Latent attention of rows [r0, r0 + Ts) -- one sequence's portion, positions pos0.. -- on the tensor-core GEMM, in blocks of query
// rows small enough that a block's score matrix stays within a fixed scratch budget.  A block only gathers the keys its rows'
// windows reach, so long prompts with short windows never touch fully masked regions.
static void latent_attn_tc(fl_cache& c, LaunchCtx& lc, const LayeredLayerW& lw, const LatentAttnArgs& a, int r0, int Ts, int pos0, int slot) {
    LayeredCache& y = *c.ly;
    const int H = a.H, C = a.C, R = a.R, E = C + R, Ep = (E + 63) / 64 * 64;
    const size_t budget = (size_t)48 << 20;                // floats in a score block (192 MB); P halves take the same again
    auto keys_for = [&](int qb, int first) {               // padded key count of the block of qb rows starting at local row `first`
        const int p_lo = pos0 + first, p_hi = pos0 + std::min(Ts, first + qb);      // positions [p_lo, p_hi)
        const int k_lo = (a.window > 0 && p_lo - a.window + 1 > 0) ? p_lo - a.window + 1 : 0;
        return ((p_hi - k_lo) + 63) / 64 * 64;
    };
    int qb = 512;
    while (qb > 8 && (size_t)qb * H * keys_for(qb, std::max(0, Ts - qb)) > budget) qb /= 2;
    const size_t rows_max = (size_t)std::min(qb, Ts) * H;
    size_t nkp_max = 0;
    for (int f = 0; f < Ts; f += qb) nkp_max = std::max<size_t>(nkp_max, keys_for(qb, f));
    auto need = [&](auto& buf, size_t n) { if (buf.n < n) { FL_CUDA(cudaStreamSynchronize(c.stream)); buf.alloc(n + n / 4); } };
    need(y.at_kc, nkp_max * Ep); need(y.at_kct, (size_t)C * nkp_max);
    need(y.at_qhi, rows_max * Ep); need(y.at_qlo, rows_max * Ep);
    need(y.at_s, rows_max * nkp_max); need(y.at_phi, rows_max * nkp_max); need(y.at_plo, rows_max * nkp_max);
    const int* page_row = y.page_table.p + (size_t)slot * c.pages_per_seq;
    for (int f = 0; f < Ts; f += qb) {
        const int nq = std::min(qb, Ts - f), p_lo = pos0 + f, p_hi = p_lo + nq;
        const int k_lo = (a.window > 0 && p_lo - a.window + 1 > 0) ? p_lo - a.window + 1 : 0, nk = p_hi - k_lo, nkp = (nk + 63) / 64 * 64;
        const int rows = nq * H;
        if (rows <= 128) {          // a short tail: the per-(row, head) kernel
            LatentAttnArgs t = a;
            t.row_base = r0 + f;
            launch_latent_attn<uint16_t>(lc, t, nq);
            continue;
        }
        launch(lc, "attn_gather_keys", 0, ly_attn_gather_keys_kernel, dim3(nkp), dim3(128), 0, (const uint16_t*)a.pool, page_row, k_lo, nk, nkp, C, E, Ep,
               y.at_kc.p, y.at_kct.p);
        launch(lc, "attn_build_q", 0, ly_attn_build_q_kernel, dim3(nq, H), dim3(128), 0, a.qa, a.proj, a.ldp, a.off_q, r0 + f, H, a.D, R, C, Ep, a.scale,
               y.at_qhi.p, y.at_qlo.p);
        const CUtensorMap tk = make_tmap_bf16(y.at_kc.p, (uint64_t)nkp, (uint64_t)Ep, (uint64_t)Ep, 128);
        dense_gemm(c, lc, "gemm_tc_attn_scores", rows, nkp, Ep, tk, y.at_s.p, y.at_qhi.p, y.at_qlo.p);
        const int keep = std::min(nkp, kSoftmaxKeep);
        launch(lc, "attn_softmax", 0, ly_attn_softmax_kernel, dim3(rows), dim3(256), (size_t)keep * 4, (const float*)y.at_s.p, a.row_pos, r0 + f, H, k_lo, 0, nk, nkp,
               a.window, 0, 0, 0.f, 0, (const float*)nullptr, keep, y.at_phi.p, y.at_plo.p);
        const CUtensorMap tv = make_tmap_bf16(y.at_kct.p, (uint64_t)C, (uint64_t)nkp, (uint64_t)nkp, 128);
        dense_gemm(c, lc, "gemm_tc_attn_values", rows, C, nkp, tv, a.ol + (size_t)(r0 + f) * H * C, y.at_phi.p, y.at_plo.p);
    }
}

// Grouped-query attention of rows [r0, r0 + Ts) -- one sequence's portion, positions pos0.. -- on the tensor-core GEMM: per block of
// query rows and per key/value head a score GEMM whose rows are (token, query head of the group) pairs, an f32 softmax (score cap,
// sink, causal mask) and a value GEMM; the block size keeps a score block within a fixed scratch budget.
static void gqa_attn_tc(fl_cache& c, LaunchCtx& lc, const GqaAttnArgs& a, int r0, int Ts, int pos0, int slot) {
    LayeredCache& y = *c.ly;
    const int H = a.H, G = a.G, rep = H / G, D = a.D, Dv = a.Dv, Dp = (D + 63) / 64 * 64, E = G * (D + Dv);
    const size_t budget = (size_t)48 << 20;                // floats in a score block (192 MB); P halves take the same again
    // first key of the contiguous range a position reads (window and chunk starts only grow with the position, so a block of
    // rows needs the keys from its first row's start on), and the kept first keys that lie before it
    auto start_of = [&](int p) {
        const int lo_w = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0, lo_c = a.chunk > 0 ? p / a.chunk * a.chunk : 0;
        return std::max(lo_w, lo_c);
    };
    auto first_of = [&](int k_lo) { return a.window > 0 ? std::min(a.keep_first, k_lo) : 0; };
    auto keys_for = [&](int qb, int first) {
        const int p_lo = pos0 + first, p_hi = pos0 + std::min(Ts, first + qb);
        const int k_lo = start_of(p_lo);
        return ((p_hi - k_lo) + first_of(k_lo) + 63) / 64 * 64;
    };
    int qb = 1024;
    while (qb > 8 && (size_t)qb * rep * keys_for(qb, std::max(0, Ts - qb)) > budget) qb /= 2;
    const size_t rows_max = (size_t)std::min(qb, Ts) * rep;
    size_t nkp_max = 0;
    for (int f = 0; f < Ts; f += qb) nkp_max = std::max<size_t>(nkp_max, keys_for(qb, f));
    auto need = [&](auto& buf, size_t n) { if (buf.n < n) { FL_CUDA(cudaStreamSynchronize(c.stream)); buf.alloc(n + n / 4); } };
    need(y.at_kc, nkp_max * Dp); need(y.at_kct, (size_t)Dv * nkp_max);
    need(y.at_qhi, rows_max * Dp); need(y.at_qlo, rows_max * Dp);
    need(y.at_s, rows_max * nkp_max); need(y.at_phi, rows_max * nkp_max); need(y.at_plo, rows_max * nkp_max);
    need(y.at_o, rows_max * G * Dv);
    const int* page_row = y.page_table.p + (size_t)slot * c.pages_per_seq;
    for (int f = 0; f < Ts; f += qb) {
        const int nq = std::min(qb, Ts - f), p_lo = pos0 + f, p_hi = p_lo + nq;
        const int k_lo = start_of(p_lo), n_first = first_of(k_lo), nk = p_hi - k_lo, nkp = (n_first + nk + 63) / 64 * 64;
        const int rows = nq * rep;
        if (rows <= 128) {          // a short tail: the per-(row, head) kernel
            GqaAttnArgs t = a;
            t.row_base = r0 + f;
            launch_gqa_attn<uint16_t>(lc, t, nq, p_hi, true);
            continue;
        }
        for (int g = 0; g < G; ++g) {
            launch(lc, "gqa_gather_kv", 0, ly_gqa_gather_kv_kernel, dim3(nkp), dim3(128), 0, (const uint16_t*)a.pool, page_row, k_lo, n_first, nk, nkp, E, g * D, D,
                   Dp, G * D + g * Dv, Dv, y.at_kc.p, y.at_kct.p);
            launch(lc, "gqa_build_q", 0, ly_gqa_build_q_kernel, dim3(nq, rep), dim3(128), 0, a.proj, a.ldp, a.off_q, r0 + f, rep, g, D, Dp, a.scale, y.at_qhi.p,
                   y.at_qlo.p);
            const CUtensorMap tk = make_tmap_bf16(y.at_kc.p, (uint64_t)nkp, (uint64_t)Dp, (uint64_t)Dp, 128);
            dense_gemm(c, lc, "gemm_tc_attn_scores", rows, nkp, Dp, tk, y.at_s.p, y.at_qhi.p, y.at_qlo.p);
            const int keep = std::min(nkp, kSoftmaxKeep);
            launch(lc, "attn_softmax", 0, ly_attn_softmax_kernel, dim3(rows), dim3(256), (size_t)keep * 4, (const float*)y.at_s.p, a.row_pos, r0 + f, rep, k_lo, n_first,
                   nk, nkp, a.window, a.keep_first, a.chunk, a.softcap, a.sink, a.sinkv ? a.sinkv + g * rep : (const float*)nullptr, keep, y.at_phi.p, y.at_plo.p);
            const CUtensorMap tv = make_tmap_bf16(y.at_kct.p, (uint64_t)Dv, (uint64_t)nkp, (uint64_t)nkp, 128);
            dense_gemm(c, lc, "gemm_tc_attn_values", rows, Dv, nkp, tv, y.at_o.p + (size_t)g * rows * Dv, y.at_phi.p, y.at_plo.p);
        }
        const size_t no = (size_t)nq * H * Dv;
        launch(lc, "gqa_scatter", 0, ly_gqa_scatter_kernel, dim3((unsigned)std::min<size_t>(4 * kNumSMs, (no + 255) / 256)), dim3(256), 0, (const float*)y.at_o.p, nq,
               G, rep, Dv, r0 + f, a.out, a.ohi, a.olo);
    }
}

static void enqueue_step(fl_cache& c, LaunchCtx& lc, const StepTab& st, const int* slots, const int* counts, int n, const int* h_row0,
                         const int* h_pos0);

void layered_forward(fl_cache& c, const int* slots, const int* counts, int n, const uint32_t* ids, const int* want, int n_want) {
    const LayeredModel& m = *c.lm;
    LayeredCache& y = *c.ly;
    FL_CHECK(!c.poisoned, FL_ERR_CUDA, "cache poisoned by an earlier CUDA error");
    FL_CHECK(slots && counts && ids && (want || n_want == 0), FL_ERR_INVALID, "NULL argument");
    FL_CHECK(n >= 1 && n <= c.max_batch && n_want >= 0, FL_ERR_INVALID, "bad batch");
    // ---- host: validate, take pages, lay out the step tables ----
    long long T = 0;
    std::vector<char> seen(c.max_batch, 0);
    int need_pages = 0;
    for (int i = 0; i < n; ++i) {
        const int sl = slots[i];
        FL_CHECK(sl >= 0 && sl < c.max_batch, FL_ERR_INVALID, "slot index out of range");
        FL_CHECK(!seen[sl], FL_ERR_INVALID, "a slot appears twice in one call");
        seen[sl] = 1;
        FL_CHECK(counts[i] >= 1, FL_ERR_INVALID, "every sequence of a step brings at least one token");
        FL_CHECK(c.slot_len[sl] + counts[i] <= c.max_seq, FL_ERR_STATE, "sequence longer than the cache's max_seq");
        FL_CHECK(m.cfg.max_positions <= 0 || c.slot_len[sl] + counts[i] <= m.cfg.max_positions, FL_ERR_STATE, "sequence longer than the model's position table");
        need_pages += y.pool.missing(sl, c.slot_len[sl] + counts[i]);
        T += counts[i];
    }
    FL_CHECK(need_pages <= y.pool.pages_free(), FL_ERR_STATE, "cache page pool exhausted");
    for (long long i = 0; i < T; ++i) FL_CHECK(ids[i] < (uint32_t)m.V, FL_ERR_INVALID, "token id out of range");
    for (int k = 0; k < n_want; ++k) FL_CHECK(want[k] >= 0 && want[k] < T, FL_ERR_INVALID, "wanted row out of range");
    ensure_ws(c, (size_t)T, (size_t)n_want);
    const size_t tab_ints = (size_t)3 * T + 3 * (size_t)n + 1 + (size_t)n_want;
    if (tab_ints > y.tab_cap) {
        FL_CUDA(cudaStreamSynchronize(c.stream));
        drop_graphs(c);
        y.tab_cap = std::max(tab_ints, 2 * y.tab_cap);
        y.step_tab.alloc(y.tab_cap); y.h_step_tab.alloc(y.tab_cap);
    }
    FL_CUDA(cudaStreamSynchronize(c.stream));      // the pinned staging buffers of the previous step are free again
    int* ht = y.h_step_tab.p;
    int *h_tok = ht, *h_rseq = ht + T, *h_rpos = ht + 2 * T, *h_row0 = ht + 3 * T, *h_slot = h_row0 + n + 1, *h_pos0 = h_slot + n,
        *h_want = h_pos0 + n;
    int row = 0;
    for (int i = 0; i < n; ++i) {
        const int sl = slots[i];
        h_row0[i] = row; h_slot[i] = sl; h_pos0[i] = c.slot_len[sl];
        for (int k = 0; k < counts[i]; ++k, ++row) { h_tok[row] = (int)ids[row]; h_rseq[row] = i; h_rpos[row] = c.slot_len[sl] + k; }
        const int before = y.pool.held(sl);
        y.pool.grow(sl, c.slot_len[sl] + counts[i]);
        if (y.pool.held(sl) != before)
            FL_CUDA(cudaMemcpyAsync(y.page_table.p + (size_t)sl * c.pages_per_seq + before, y.pool.row(sl) + before,
                                    (size_t)(y.pool.held(sl) - before) * 4, cudaMemcpyHostToDevice, c.stream));
    }
    h_row0[n] = row;
    for (int k = 0; k < n_want; ++k) h_want[k] = want[k];
    FL_CUDA(cudaMemcpyAsync(y.step_tab.p, ht, tab_ints * 4, cudaMemcpyHostToDevice, c.stream));
    const int* dt = y.step_tab.p;
    StepTab st{dt, dt + T, dt + 2 * T, dt + 3 * T, dt + 3 * T + n + 1, dt + 3 * T + 2 * n + 1, dt + 3 * T + 3 * n + 1, (int)T, n, n_want};

    // ---- device: layer by layer over all rows of the step ----
    LaunchCtx lc;
    lc.stream = c.stream;
    lc.pdl = false;
    lc.exact = m.f32;
    // A step in which every sequence brings ONE token has a launch geometry that depends on (sequences, wanted rows) alone --
    // positions, slots and pages are read from the device tables -- so it is captured into a CUDA graph the second time the pair is
    // seen and replayed from then on (FL_NO_GRAPH=1 keeps eager launches).
    static const bool no_graph = env_flag("FL_NO_GRAPH");
    if (T == n && !g_prof.on && !no_graph) {
        const GraphKey key{n, 1000 + n_want};
        auto it = c.graphs.find(key);
        if (it == c.graphs.end()) {
            c.graphs[key] = GraphEntry{};               // first sight: run eagerly (one-time kernel attributes, lazy loading)
            enqueue_step(c, lc, st, slots, counts, n, h_row0, h_pos0);
        } else {
            if (it->second.exec == nullptr) {
                lc.capturing = true;
                cudaGraph_t graph = nullptr;
                FL_CUDA(cudaStreamBeginCapture(c.stream, cudaStreamCaptureModeThreadLocal));
                try {
                    enqueue_step(c, lc, st, slots, counts, n, h_row0, h_pos0);
                } catch (...) {
                    cudaStreamEndCapture(c.stream, &graph);
                    if (graph) cudaGraphDestroy(graph);
                    throw;
                }
                FL_CUDA(cudaStreamEndCapture(c.stream, &graph));
                GraphEntry e;
                FL_CUDA(cudaGraphInstantiate(&e.exec, graph, 0));
                FL_CUDA(cudaGraphDestroy(graph));
                e.kernels = lc.captured;
                it->second = e;
            }
            FL_CUDA(cudaGraphLaunch(it->second.exec, c.stream));
            g_launches.fetch_add(it->second.kernels, std::memory_order_relaxed);
        }
    } else {
        enqueue_step(c, lc, st, slots, counts, n, h_row0, h_pos0);
    }
    if (n_want > 0)
        FL_CUDA(cudaMemcpyAsync(y.h_logits.p, y.logits.p, (size_t)n_want * m.V * 4, cudaMemcpyDeviceToHost, c.stream));
    for (int i = 0; i < n; ++i) c.slot_len[slots[i]] += counts[i];
}

// One mixer over all rows of the step: reads its columns of the projected buffer y.proj (row stride lw.n_in), its cache pages / state
// slots, and leaves the mixer's inner output (what its output projection reads) in y.u with the hi | lo halves when that
// projection runs on the tensor cores.
static void run_mixer(fl_cache& c, LaunchCtx& lc, const StepTab& st, const LayeredLayerW& lw, const int* slots, const int* counts, int n,
                      const int* h_row0, const int* h_pos0) {
    const LayeredModel& m = *c.lm;
    LayeredCache& y = *c.ly;
    const fl_layer_desc& d = lw.d;
    const int Ti = st.T, H = d.heads, D = d.dim, Dv = d.vdim;
    const float eps = m.cfg.norm_eps;
    uint16_t *uhi = m.f32 ? nullptr : y.u_hi.p, *ulo = m.f32 ? nullptr : y.u_lo.p;
    if (d.mixer == FL_MIXER_ATTN) {
        const int G = d.kv_heads;
        AttnPrepArgs pa{y.proj.p, lw.n_in, lw.off_q, lw.off_k, lw.off_v, lw.qnorm, lw.knorm, eps, y.kv_pool[lw.kv_index], y.page_table.p,
                        c.pages_per_seq, st.row_seq, st.row_pos, st.seq_slot, y.rope_cos[lw.rope_index].p, y.rope_sin[lw.rope_index].p,
                        H, G, D, Dv, d.rot_dims, d.rot_halves, lw.bq, lw.bk, lw.bv, d.qk_norm_whole};
        // eight warps per block take the heads in turn; steps of few rows spread a row's heads over up to four blocks (not with a
        // norm over the whole projection: its sums read every head before any is rewritten in place, which one block orders)
        const size_t psm = (size_t)8 * D * 4;
        const int heads_all = H + (lw.off_k >= 0 ? G : 0), py = (Ti <= 64 && !d.qk_norm_whole) ? std::max(1, std::min(4, (heads_all + 7) / 8)) : 1;
        if (m.f32) launch(lc, "attn_prep", 0, ly_attn_prep_kernel<float>, dim3(Ti, py), dim3(256), psm, pa);
        else launch(lc, "attn_prep", 0, ly_attn_prep_kernel<uint16_t>, dim3(Ti, py), dim3(256), psm, pa);
        GqaAttnArgs at{y.proj.p, lw.n_in, lw.off_q, y.kv_pool[lw.kv_index], y.page_table.p, c.pages_per_seq, st.row_seq, st.row_pos, st.seq_slot,
                       y.u.p, lw.tc_o ? uhi : (uint16_t*)nullptr, ulo, H, G, D, Dv, d.window, d.scale, d.softcap, d.sink, 0, y.at_part.p,
                       d.keep_first, d.mask_chunk, lw.sinkv};
        // a step of single tokens is replayed from a captured graph whatever the contexts' lengths: its split count must not follow them
        int max_keys = c.max_seq;
        if (Ti != n) {
            max_keys = 1;
            for (int si = 0; si < n; ++si) max_keys = std::max(max_keys, h_pos0[si] + counts[si]);
        }
        if (d.window > 0) max_keys = std::min(max_keys, d.window + d.keep_first);
        if (d.mask_chunk > 0) max_keys = std::min(max_keys, d.mask_chunk);
        // masks that leave a row few keys: the per-row kernel reads just those, the GEMM path would compute a block's whole rectangle
        const bool few_keys = (d.window > 0 && d.window + d.keep_first <= 256) || (d.mask_chunk > 0 && d.mask_chunk <= 256);
        // long portions (serving precision): scores and weighted sums as tensor-core GEMMs; decoded tokens, short portions and
        // the exact mode on the per-(row, head) kernel.  Rows are taken in order.
        static const bool tc_attn_off = env_flag("FL_LAYERED_NO_TC_ATTN");
        int done = 0;
        for (int si = 0; si < n; ++si) {
            const int r0 = h_row0[si], Ts = counts[si];
            if (m.f32 || tc_attn_off || few_keys || Dv % 8 != 0 || Ts < 64 || (long long)Ts * (H / G) <= 128) continue;
            if (r0 > done) {
                at.row_base = done;
                launch_gqa_attn<uint16_t>(lc, at, r0 - done, max_keys, true);
            }
            gqa_attn_tc(c, lc, at, r0, Ts, h_pos0[si], slots[si]);
            done = r0 + Ts;
        }
        if (done < Ti) {
            at.row_base = done;
            if (m.f32) launch_gqa_attn<float>(lc, at, Ti - done, max_keys, false); else launch_gqa_attn<uint16_t>(lc, at, Ti - done, max_keys, true);
        }
    } else if (d.mixer == FL_MIXER_MAMBA2 || d.mixer == FL_MIXER_DELTA) {
        const bool delta = d.mixer == FL_MIXER_DELTA;
        const int G = delta ? d.kv_heads : d.groups, rows = delta ? D : d.state;
        float* cstate = d.conv > 1 ? y.conv_state[lw.gla_index].p : nullptr;
        ConvArgs ca{y.proj.p, lw.n_in, lw.conv_off, lw.conv_w, lw.conv_b, cstate, st.row_seq, st.row_pos, st.seq_row0, st.seq_slot, st.seq_pos0,
                    lw.conv_ch, d.conv, y.cv.p};
        // channel chunks per row: whole q / k heads for the delta rule (they are normalised inside one block)
        const int chunk = delta ? D * std::max(1, 512 / D) : 512, nchunk = (lw.conv_ch + chunk - 1) / chunk;
        if (delta)
            launch(lc, "delta_prep", 0, ly_delta_prep_kernel, dim3(Ti, nchunk), dim3(256), 0, ca, chunk, lw.off_b, lw.off_a, (const float*)lw.dt_bias,
                   (const float*)lw.a_log, H, G, D, (float)(1.0 / std::sqrt((double)D)), y.rs.p);
        else
            launch(lc, "ssm_prep", 0, ly_mamba_prep_kernel, dim3(Ti, nchunk), dim3(256), 0, ca, chunk, lw.off_dt, (const float*)lw.dt_bias,
                   (const float*)lw.a_log, H, y.rs.p);
        if (d.conv > 1) launch(lc, "conv_state", 0, ly_conv_state_kernel, dim3(n, (lw.conv_ch + 127) / 128), dim3(128), 0, ca);
        // column offsets inside cv (the convolved span starts at conv_off)
        RecArgs ra{y.cv.p, lw.conv_ch, lw.off_q - lw.conv_off, lw.off_k - lw.conv_off, lw.off_v - lw.conv_off, y.rs.p,
                   delta ? (const float*)nullptr : (const float*)lw.dskip, y.go.p, y.gla_state[lw.gla_index].p, st.seq_row0, st.seq_slot, st.seq_pos0,
                   H, G, rows, Dv};
        if (delta) {
            launch_rec_scan<true>(lc, ra, n);
            launch(lc, "gla_out", 0, ly_gla_out_kernel, dim3((Ti * H + 7) / 8), dim3(256), 0, (const float*)y.go.p, (const float*)y.proj.p, lw.n_in, lw.off_g,
                   (const float*)lw.hnorm, eps, Ti, H, Dv, y.u.p, lw.tc_o ? uhi : (uint16_t*)nullptr, ulo);
        } else {
            launch_rec_scan<false>(lc, ra, n);
            const int inner = H * Dv, part = inner / d.norm_groups;
            launch(lc, "gated_group_norm", 0, ly_gated_group_norm_kernel, dim3(Ti, d.norm_groups), dim3(std::min(1024, std::max(64, (part + 31) / 32 * 32))), 0,
                   (const float*)y.go.p, (const float*)y.proj.p, lw.n_in, lw.off_g, (const float*)lw.hnorm, eps, inner, d.norm_groups, 0, y.u.p,
                   lw.tc_o ? uhi : (uint16_t*)nullptr, ulo);
        }
    } else if (d.mixer == FL_MIXER_LIGHTNING) {
        const int chunk = 512, nchunk = (lw.conv_ch + chunk - 1) / chunk, inner = H * Dv;
        launch(lc, "lightning_prep", 0, ly_lightning_prep_kernel, dim3(Ti, nchunk), dim3(256), 0, (const float*)y.proj.p, lw.n_in, lw.conv_off, lw.conv_ch, chunk,
               (const float*)lw.decay, H, y.cv.p, y.rs.p);
        RecArgs ra{y.cv.p, lw.conv_ch, lw.off_q - lw.conv_off, lw.off_k - lw.conv_off, lw.off_v - lw.conv_off, y.rs.p, (const float*)nullptr, y.go.p,
                   y.gla_state[lw.gla_index].p, st.seq_row0, st.seq_slot, st.seq_pos0, H, H, D, Dv};
        launch_rec_scan<false>(lc, ra, n);
        const bool v4 = ((inner | lw.n_in | lw.off_g) & 3) == 0;       // four channels per thread
        launch(lc, "gated_group_norm", 0, ly_gated_group_norm_kernel, dim3(Ti, 1), dim3(std::min(v4 ? 256 : 1024, std::max(64, ((v4 ? inner / 4 : inner) + 31) / 32 * 32))), 0,
               (const float*)y.go.p, (const float*)y.proj.p, lw.n_in, lw.off_g, (const float*)lw.hnorm, eps, inner, 1, 1, y.u.p,
               lw.tc_o ? uhi : (uint16_t*)nullptr, ulo);
    } else if (d.mixer == FL_MIXER_GLA) {
        // decay pre-activation through the rank-r bottleneck: z = W_a2 a (the bias and the sigmoid^(1/tau) are applied by the scan)
        gemm(lc, "gemm_gla_decay", y.proj.p + lw.off_a, lw.n_in, lw.a2, H * D, d.decay_rank, y.la.p, H * D, Ti);
        GlaArgs ga{y.proj.p, lw.n_in, lw.off_q, lw.off_k, lw.off_v, y.la.p, lw.a2b, 1.f / d.tau, y.go.p, y.gla_state[lw.gla_index].p, st.seq_row0,
                   st.seq_slot, st.seq_pos0, H, D, Dv, (float)(1.0 / std::sqrt((double)D))};
        launch_gla_scan(lc, ga, n);
        launch(lc, "gla_out", 0, ly_gla_out_kernel, dim3((Ti * H + 7) / 8), dim3(256), 0, (const float*)ga.o, (const float*)y.proj.p, lw.n_in, lw.off_g,
               (const float*)lw.hnorm, eps, Ti, H, Dv, y.u.p, lw.tc_o ? uhi : (uint16_t*)nullptr, ulo);
    } else {
        const int R = d.rot_dim, C = d.kv_rank;
        LatentAppendArgs aa{y.proj.p, lw.n_in, lw.off_q, lw.off_dkv, lw.dkv_norm, eps, y.kv_pool[lw.kv_index], y.page_table.p, c.pages_per_seq,
                            st.row_seq, st.row_pos, st.seq_slot, y.rope_cos[lw.rope_index].p, y.rope_sin[lw.rope_index].p, H, D, R, C, d.rot_dims};
        if (m.f32) launch(lc, "latent_append", 0, ly_latent_append_kernel<float>, dim3(Ti), dim3(128), 0, aa);
        else launch(lc, "latent_append", 0, ly_latent_append_kernel<uint16_t>, dim3(Ti), dim3(128), 0, aa);
        // q~[row, h, :] = W_uk[h]^T q_plain[row, h, :]: the score against the latent needs no per-head keys
        LyGemm qa{y.proj.p + lw.off_q, D + R, lw.n_in, nullptr, lw.uk_t, (long long)C * D, C, D, y.qa.p, C, H * C, nullptr, Ti};
        gemm_groups(lc, "gemm_q_absorb", qa, H, Ti);
        LatentAttnArgs at{y.qa.p, y.proj.p, lw.n_in, lw.off_q, y.kv_pool[lw.kv_index], y.page_table.p, c.pages_per_seq, st.row_seq, st.row_pos,
                          st.seq_slot, y.ol.p, H, D, R, C, d.window, d.scale, 0};
        // long portions (serving precision): scores and weighted sums as tensor-core GEMMs over the gathered window; everything
        // else (decoded tokens, short portions, the exact mode) on the per-(row, head) kernel.  Rows are taken in order.
        static const bool tc_attn_off = env_flag("FL_LAYERED_NO_TC_ATTN");
        int done = 0;           // rows [0, done) are finished
        for (int si = 0; si < n; ++si) {
            const int r0 = h_row0[si], Ts = counts[si];
            if (m.f32 || tc_attn_off || C % 8 != 0 || Ts < 64 || (long long)Ts * H <= 128) continue;
            if (r0 > done) {
                at.row_base = done;
                launch_latent_attn<uint16_t>(lc, at, r0 - done);
            }
            latent_attn_tc(c, lc, lw, at, r0, Ts, h_pos0[si], slots[si]);
            done = r0 + Ts;
        }
        if (done < Ti) {
            at.row_base = done;
            if (m.f32) launch_latent_attn<float>(lc, at, Ti - done); else launch_latent_attn<uint16_t>(lc, at, Ti - done);
        }
        // value expansion after the softmax: out[row, h, :] = W_uv[h] (sum_j p_j c_j)
        LyGemm ov{y.ol.p, C, H * C, nullptr, lw.uv, (long long)Dv * C, Dv, C, y.u.p, Dv, H * Dv, nullptr, Ti};
        gemm_groups(lc, "gemm_v_expand", ov, H, Ti);
        if (lw.tc_o) {
            const size_t nu = (size_t)Ti * H * Dv;
            launch(lc, "split_hi_lo", 0, ly_split_kernel, dim3((unsigned)std::min<size_t>(4 * kNumSMs, (nu + 255) / 256)), dim3(256), 0,
                   (const float*)y.u.p, nu, uhi, ulo);
        }
    }
}

// The device part of a step: every layer over all rows, then the vocabulary projection of the wanted rows.
static void enqueue_step(fl_cache& c, LaunchCtx& lc, const StepTab& st, const int* slots, const int* counts, int n, const int* h_row0,
                         const int* h_pos0) {
    const LayeredModel& m = *c.lm;
    LayeredCache& y = *c.ly;
    const int n_want = st.n_want;
    const int Ti = st.T, W = m.W;
    const float eps = m.cfg.norm_eps;
    const int nthr = std::min(1024, std::max(64, (W + 31) / 32 * 32));
    uint16_t *hhi = m.f32 ? nullptr : y.h_hi.p, *hlo = m.f32 ? nullptr : y.h_lo.p, *uhi = m.f32 ? nullptr : y.u_hi.p, *ulo = m.f32 ? nullptr : y.u_lo.p,
             *ahi = m.f32 ? nullptr : y.act_hi.p, *alo = m.f32 ? nullptr : y.act_lo.p;
    // pre-norm stacks: a sublayer reads h = norm(x) (written by the kernel that last touched x); otherwise it reads x itself and
    // the same kernel writes x's hi | lo halves for the tensor-core GEMMs.  With an input convolution the sublayer reads
    // hc = h + conv(h) instead (the convolution kernel rewrites the hi | lo halves after the gate's GEMM has read those of h).
    const bool pre = !m.cfg.no_pre_norm, post = !m.cfg.no_post_norm, canon = m.cfg.canon_taps > 0, gated = m.cfg.gated_residual != 0,
               depth = m.cfg.depth_avg != 0;
    const int plain = m.cfg.norm_plain ? 1 : 0, split_x = pre ? 0 : 1;
    const float* norm_out = pre ? y.h.p : y.x.p;                // what the arrangement hands to a sublayer
    const float* sub_in = canon ? y.hc.p : norm_out;            // what the sublayer's own matrices read
    const size_t hist_stride = y.rows * (size_t)W;
    launch(lc, "embed_norm", 0, ly_embed_norm_kernel, dim3(Ti), dim3(nthr), 0, (const uint16_t*)m.embed, st.tok, W,
           pre ? (const float*)m.layers[0].norm1 : (const float*)nullptr, eps, plain, (const uint16_t*)m.pos, st.row_pos, m.cfg.embed_scale, y.x.p,
           depth ? y.xs.p : (float*)nullptr, y.h.p, hhi, hlo);
    // in front of a sublayer: the gate's pre-activation from the normed input, then the input convolution (and its carried inputs)
    auto sublayer_front = [&](const LayeredLayerW& lw, int sub) {
        if (gated) {
            const uint16_t* rg = sub == 0 ? lw.rg1 : lw.rg2;
            gemm_tc_or_exact(c, lc, "gemm_gate", norm_out, hhi, hlo, rg, sub == 0 ? lw.tm_rg1 : lw.tm_rg2, sub == 0 ? lw.tc_rg1 : lw.tc_rg2, W, W, y.gz.p, Ti);
        }
        if (canon) {
            const int taps = m.cfg.canon_taps;
            float* cs = taps > 1 ? y.canon_state[lw.canon_index].p + (size_t)sub * c.max_batch * (taps - 1) * W : nullptr;
            ConvArgs ca{norm_out, W, 0, sub == 0 ? lw.canon1 : lw.canon2, nullptr, cs, st.row_seq, st.row_pos, st.seq_row0, st.seq_slot, st.seq_pos0, W, taps, nullptr};
            // few rows: one row per block; long steps: a block walks 8 rows with its taps staged once
            const int rpb = Ti >= 1024 ? 8 : 1;
            if (W % 4 == 0)
                launch(lc, "input_conv", 0, ly_input_conv_kernel<4>, dim3((Ti + rpb - 1) / rpb, (W / 4 + 127) / 128), dim3(128), (size_t)taps * 128 * 4 * 4, ca, rpb, Ti,
                       y.hc.p, hhi, hlo);
            else
                launch(lc, "input_conv", 0, ly_input_conv_kernel<1>, dim3((Ti + rpb - 1) / rpb, (W + 127) / 128), dim3(128), (size_t)taps * 128 * 4, ca, rpb, Ti,
                       y.hc.p, hhi, hlo);
            if (taps > 1) launch(lc, "conv_state", 0, ly_conv_state_kernel, dim3(n, (W + 127) / 128), dim3(128), 0, ca);
        }
    };
    // stacks with a token shift: the mixer reads hc = x + (x_prev - x) * shift (x_prev from the row before, or the slot's carried
    // row); the slot then keeps this step's last row of x.  The shift kernel rewrites the hi | lo halves with those of hc.
    const bool shifted = m.cfg.token_shift != 0, sum_norm = m.cfg.post_sum_norm != 0;
    auto shift_front = [&](const LayeredLayerW& lw, int li) {
        ConvArgs ca{y.x.p, W, 0, nullptr, nullptr, y.shift_state[li].p, st.row_seq, st.row_pos, st.seq_row0, st.seq_slot, st.seq_pos0, W, 2, nullptr};
        if (W % 4 == 0)
            launch(lc, "token_shift", 0, ly_token_shift_kernel<4>, dim3(Ti, (W / 4 + 127) / 128), dim3(128), 0, ca, (const float*)lw.shift, y.hc.p, hhi, hlo);
        else
            launch(lc, "token_shift", 0, ly_token_shift_kernel<1>, dim3(Ti, (W + 127) / 128), dim3(128), 0, ca, (const float*)lw.shift, y.hc.p, hhi, hlo);
        launch(lc, "conv_state", 0, ly_conv_state_kernel, dim3(n, (W + 127) / 128), dim3(128), 0, ca);
    };
    // the norm of the sum: x <- norm(alpha x + sa y (+ sb y2)); split: whether another sublayer reads the new x through the tensor cores
    auto sum_norm_join = [&](const float* yb, const float* y2, float sa, float sb, const float* w, int split) {
        if (W % 4 == 0)
            launch(lc, "sum_norm", 0, ly_sum_norm_kernel<4>, dim3(Ti), dim3(std::min(256, std::max(32, (W / 4 + 31) / 32 * 32))), (size_t)W * 4, y.x.p,
                   (const float*)y.y.p, yb, y2, m.cfg.residual_alpha, sa, sb, w, eps, W, plain, split, hhi, hlo);
        else
            launch(lc, "sum_norm", 0, ly_sum_norm_kernel<1>, dim3(Ti), dim3(nthr), (size_t)W * 4, y.x.p, (const float*)y.y.p, yb, y2, m.cfg.residual_alpha, sa, sb,
                   w, eps, W, plain, split, hhi, hlo);
    };
    // a sublayer's result (y.y, and y2 beside it) joins the stream; four channels per thread when the rows are 16-byte multiples
    auto join = [&](const float* y2, const float* wa, const float* wb, const float* gate_bias, int hist_slot, const float* dw, const float* wnext) {
        const float* gz = gated ? (const float*)y.gz.p : (const float*)nullptr;
        if (W % 4 == 0)
            launch(lc, "join", 0, ly_join_kernel<4>, dim3(Ti), dim3(std::min(256, std::max(32, (W / 4 + 31) / 32 * 32))), 0, y.x.p, (const float*)y.y.p, y2, wa, wb,
                   gz, gate_bias, y.xs.p, hist_stride, hist_slot, dw, wnext, eps, W, plain, y.h.p, hhi, hlo);
        else
            launch(lc, "join", 0, ly_join_kernel<1>, dim3(Ti), dim3(nthr), 0, y.x.p, (const float*)y.y.p, y2, wa, wb, gz, gate_bias, y.xs.p, hist_stride,
                   hist_slot, dw, wnext, eps, W, plain, y.h.p, hhi, hlo);
    };
    for (int li = 0; li < m.L; ++li) {
        const LayeredLayerW& lw = m.layers[li];
        const fl_layer_desc& d = lw.d;
        const int H = d.heads, Dv = d.vdim;
        sublayer_front(lw, 0);
        if (shifted) shift_front(lw, li);
        gemm_tc_or_exact(c, lc, "gemm_mix_in", shifted ? (const float*)y.hc.p : sub_in, hhi, hlo, lw.w_in, lw.tm_in, lw.tc_in, lw.n_in, W, y.proj.p, Ti);
        run_mixer(c, lc, st, lw, slots, counts, n, h_row0, h_pos0);
        gemm_tc_or_exact(c, lc, "gemm_mix_out", y.u.p, uhi, ulo, lw.w_o, lw.tm_o, lw.tc_o, W, H * Dv, y.y.p, Ti);
        if (lw.side) {
            const LayeredLayerW& sw = *lw.side;
            run_mixer(c, lc, st, sw, slots, counts, n, h_row0, h_pos0);
            gemm_tc_or_exact(c, lc, "gemm_mix_out", y.u.p, uhi, ulo, sw.w_o, sw.tm_o, sw.tc_o, W, sw.d.heads * sw.d.vdim, y.y2.p, Ti);
        }
        const float* next1 = (pre && li + 1 < m.L) ? m.layers[li + 1].norm1 : nullptr;
        const int more = li + 1 < m.L ? split_x : 0;       // whether another sublayer reads x after this layer
        const bool has_ff = d.ffn != FL_FFN_NONE;
        if (sum_norm)
            sum_norm_join(nullptr, lw.side ? (const float*)y.y2.p : (const float*)nullptr, lw.side ? d.out_scale : 1.f, lw.side ? lw.side->d.out_scale : 0.f,
                          lw.norm1b, (has_ff || !shifted) ? (has_ff ? split_x : more) : 0);
        else if (post)
            launch(lc, "post_norm", 0, ly_post_norm_kernel, dim3(Ti), dim3(nthr), 0, y.x.p, (const float*)y.y.p, (const float*)nullptr, (const float*)lw.norm1b,
                   has_ff ? (const float*)lw.norm2 : next1, eps, W, plain, has_ff ? split_x : more, y.h.p, hhi, hlo);
        else
            join(lw.side ? (const float*)y.y2.p : (const float*)nullptr, lw.pair_wa, lw.pair_wb, lw.rg1b, (depth && !has_ff) ? li + 1 : -1, lw.dwa,
                 has_ff ? (const float*)lw.norm2 : next1);
        if (!has_ff) continue;
        sublayer_front(lw, 1);
        const int F = d.ff, act = d.ffn_act, GF = act == FL_ACT_RELU2 ? F : 2 * F;
        if (d.ffn == FL_FFN_DENSE) {
            gemm_tc_or_exact(c, lc, "gemm_ff_in", sub_in, hhi, hlo, lw.w_gu, lw.tm_gu, lw.tc_gu, GF, W, y.gu.p, Ti);
            launch(lc, "glu", 0, ly_glu_kernel, dim3(std::min(4 * kNumSMs, (Ti * F + 255) / 256)), dim3(256), 0, (const float*)y.gu.p, F, d.limit,
                   act, (const float*)lw.b_gu, (const int*)nullptr, Ti, lw.tc_down ? (float*)nullptr : y.act.p, lw.tc_down ? ahi : (uint16_t*)nullptr, alo);
            gemm_tc_or_exact(c, lc, "gemm_ff_out", y.act.p, ahi, alo, lw.w_down, lw.tm_down, lw.tc_down, W, F, y.y.p, Ti);
        } else {
            const int E = d.experts, top = d.top, P = Ti * top;
            if (d.router == FL_ROUTER_SIGMOID_GROUPS)
                launch(lc, "moe_router", 0, ly_router_sigmoid_kernel, dim3(Ti), dim3(256), ((size_t)2 * E + d.route_groups) * 4, sub_in, W, (const float*)lw.router,
                       E, top, (const float*)lw.route_corr, d.route_groups, d.route_keep, y.route_sel.p, y.route_w.p);
            else
                launch(lc, "moe_router", 0, ly_router_kernel, dim3(Ti), dim3(256), (size_t)E * 4, sub_in, W, (const float*)lw.router, (const float*)lw.router_b, E, top,
                       (const float*)lw.shared_gate, y.route_sel.p, y.route_w.p, y.sgate.p);
            const float* sg = lw.shared_gate ? (const float*)y.sgate.p : (const float*)nullptr;    // nullptr: the shared expert counts fully
            const float* sh = nullptr;
            if (d.shared_ff > 0) {          // the always-on expert first: its split-K scratch is free again before the routed experts run
                const int Fs = d.shared_ff;
                gemm_tc_or_exact(c, lc, "gemm_shared_in", sub_in, hhi, hlo, lw.s_gu, lw.tm_sgu, lw.tc_sgu, 2 * Fs, W, y.sh_gu.p, Ti);
                launch(lc, "glu", 0, ly_glu_kernel, dim3(std::min(4 * kNumSMs, (Ti * Fs + 255) / 256)), dim3(256), 0, (const float*)y.sh_gu.p, Fs,
                       d.shared_limit, 0, (const float*)nullptr, (const int*)nullptr, Ti, lw.tc_sdown ? (float*)nullptr : y.sh_act.p, lw.tc_sdown ? ahi : (uint16_t*)nullptr, alo);
                gemm_tc_or_exact(c, lc, "gemm_shared_out", y.sh_act.p, ahi, alo, lw.s_down, lw.tm_sdown, lw.tc_sdown, W, Fs, y.sh_o.p, Ti);
                sh = y.sh_o.p;
            }
            const dim3 gw((W + 255) / 256, Ti);
            if (lw.tc_moe && Ti > 128) {
                // many rows: every expert over all rows on the tensor cores, kept where the row picked it (ascending expert order)
                for (int e = 0; e < E; ++e) {
                    dense_gemm(c, lc, "gemm_tc_moe_in", Ti, GF, W, lw.tm_egu[e], y.gu.p, hhi, hlo);
                    launch(lc, "glu", 0, ly_glu_kernel, dim3(std::min(4 * kNumSMs, (Ti * F + 255) / 256)), dim3(256), 0, (const float*)y.gu.p, F, d.limit,
                           act, (const float*)nullptr, (const int*)nullptr, Ti, (float*)nullptr, ahi, alo);
                    dense_gemm(c, lc, "gemm_tc_moe_out", Ti, W, F, lw.tm_edown[e], y.eo.p, ahi, alo);
                    launch(lc, "moe_accum", 0, ly_moe_accum_kernel, gw, dim3(256), 0, (const float*)y.eo.p, (const int*)y.route_sel.p,
                           (const float*)y.route_w.p, top, e, (const float*)nullptr, e == 0 ? 1 : 0, W, y.y.p);
                }
                if (sh != nullptr)
                    launch(lc, "moe_accum", 0, ly_moe_accum_kernel, gw, dim3(256), 0, sh, (const int*)nullptr, (const float*)nullptr, 0, -1,
                           sg, 0, W, y.y.p);
            } else {
                launch(lc, "moe_lists", 0, ly_moe_lists_kernel, dim3(E), dim3(32), 0, (const int*)y.route_sel.p, Ti, top, E, y.grp_off.p, y.pair_row.p,
                       y.pair_of.p);
                if (lw.tc_moe) {
                    // few rows: ONE grouped GEMM pair over (expert, weight tile, k slice) items; an expert without rows costs nothing
                    const int cap = Ti <= 16 ? 16 : (Ti <= 32 ? 32 : (Ti <= 64 ? 64 : 128));
                    launch(lc, "moe_gather", 0, ly_moe_gather_kernel, dim3(E, std::min(Ti, 16)), dim3(256), 0, (const uint16_t*)hhi, (const uint16_t*)hlo, W,
                           (const int*)y.grp_off.p, (const int*)y.pair_row.p, cap, y.gx_hi.p, y.gx_lo.p, y.grp_cnt.p);
                    int ks = dense_gemm_grouped(c, lc, "gemm_tc_moe_in", E, cap, GF, W, lw.tm_gu, y.gemm_out.p, y.gx_hi.p, y.gx_lo.p, y.grp_cnt.p);
                    FL_CHECK((size_t)ks * E * cap * GF <= y.gemm_out.n, FL_ERR_STATE, "internal: grouped GEMM scratch too small");
                    launch(lc, "glu_grouped", 0, ly_glu_grouped_kernel, dim3((F + 255) / 256, E * cap), dim3(256), 0, (const float*)y.gemm_out.p, ks,
                           (size_t)E * cap * GF, F, d.limit, act, (const int*)y.grp_cnt.p, cap, y.ga_hi.p, y.ga_lo.p);
                    ks = dense_gemm_grouped(c, lc, "gemm_tc_moe_out", E, cap, W, F, lw.tm_down, y.gemm_out.p, y.ga_hi.p, y.ga_lo.p, y.grp_cnt.p);
                    FL_CHECK((size_t)ks * E * cap * W <= y.gemm_out.n, FL_ERR_STATE, "internal: grouped GEMM scratch too small");
                    launch(lc, "moe_combine", 0, ly_moe_combine_grouped_kernel, gw, dim3(256), 0, (const float*)y.gemm_out.p, ks, (size_t)E * cap * W,
                           (const int*)y.route_sel.p, (const int*)y.pair_of.p, (const int*)y.grp_off.p, cap, (const float*)y.route_w.p, top, sh,
                           sg, W, y.y.p);
                } else {
                    LyGemm g1{sub_in, 0, W, y.pair_row.p, lw.w_gu, (long long)GF * W, GF, W, y.gu.p, 0, GF, y.grp_off.p, P};
                    gemm_groups(lc, "gemm_moe_in", g1, E, P);
                    launch(lc, "glu", 0, ly_glu_kernel, dim3(std::min(4 * kNumSMs, (P * F + 255) / 256)), dim3(256), 0, (const float*)y.gu.p, F, d.limit,
                           act, (const float*)nullptr, (const int*)nullptr, P, y.act.p, (uint16_t*)nullptr, (uint16_t*)nullptr);
                    LyGemm g2{y.act.p, 0, F, nullptr, lw.w_down, (long long)W * F, W, F, y.eo.p, 0, W, y.grp_off.p, P};
                    gemm_groups(lc, "gemm_moe_out", g2, E, P);
                    launch(lc, "moe_combine", 0, ly_moe_combine_kernel, gw, dim3(256), 0, (const float*)y.eo.p, (const int*)y.pair_of.p,
                           (const float*)y.route_w.p, top, sh, sg, W, y.y.p);
                }
            }
        }
        if (sum_norm)
            sum_norm_join(lw.b_down, nullptr, 1.f, 0.f, lw.norm2b, shifted ? 0 : more);
        else if (post)
            launch(lc, "post_norm", 0, ly_post_norm_kernel, dim3(Ti), dim3(nthr), 0, y.x.p, (const float*)y.y.p, (const float*)lw.b_down, (const float*)lw.norm2b,
                   next1, eps, W, plain, more, y.h.p, hhi, hlo);
        else
            join(nullptr, nullptr, nullptr, lw.rg2b, depth ? li + 1 : -1, lw.dwa, next1);
    }
    if (n_want > 0) {
        launch(lc, "final_norm", 0, ly_final_norm_kernel, dim3(n_want), dim3(nthr), 0, (const float*)y.x.p, st.want, (const float*)m.final_norm, eps, W, plain, y.hf.p,
               m.tc_head ? y.hf_hi.p : (uint16_t*)nullptr, y.hf_lo.p);
        gemm_tc_or_exact(c, lc, "gemm_head", y.hf.p, m.tc_head ? y.hf_hi.p : nullptr, y.hf_lo.p, m.head, m.tm_head, m.tc_head, m.V, W, y.logits.p, n_want);
        if (m.cfg.logit_softcap > 0.f) {
            const size_t nl = (size_t)n_want * m.V;
            launch(lc, "logit_cap", 0, ly_softcap_kernel, dim3((unsigned)std::min<size_t>(4 * kNumSMs, (nl + 255) / 256)), dim3(256), 0, y.logits.p, nl,
                   m.cfg.logit_softcap);
        }
    }
}

}  // namespace fl
