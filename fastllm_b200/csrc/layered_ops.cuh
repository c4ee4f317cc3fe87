// Kernels of the layered decoders (sm_100a): residual / norm glue, the exact-f32 GEMM, gated linear attention (decay, scan, head
// norm + gate), latent attention over the paged latent cache (append + rotary, absorbed-query attention), grouped-query attention
// with per-head q/k norm, score cap and softmax sink, the short-convolution recurrent mixers (Mamba-2, gated delta rule: prep, scan,
// gated norms), the feed-forward (clamped swish or tanh-gelu GLU with optional biases, ungated squared relu), the mixture-of-experts
// routers (softmax top-k; sigmoid scores with a choice correction and group-limited choice) / row lists / combine, and the pieces of
// stacks whose sublayer results join the stream un-normed (learned positions, input convolution, gated contribution, two mixers
// side by side, depth average).  Every mechanism takes its sizes and constants as
// arguments.  Residual stream, norms, softmax, routers, decays and the recurrent state are f32 throughout; a row's result never
// depends on which other rows share the launch (fixed summation order per output element).
#pragma once
#include <math.h>

#include "common.cuh"
#include "mma.cuh"

namespace fl {

// ---- per-step integer tables (one upload per step) -------------------------------------------------------------------------
struct StepTab {
    const int* tok;         // [T] token id of every row
    const int* row_seq;     // [T] index of the row's sequence inside this step
    const int* row_pos;     // [T] position of the row inside its sequence
    const int* seq_row0;    // [n + 1] first row of every sequence
    const int* seq_slot;    // [n] cache slot
    const int* seq_pos0;    // [n] tokens the slot held before this step
    const int* want;        // [n_want] rows whose logits are asked for
    int T, n, n_want;
};

// cache element: float (exact mode) or bf16 bit pattern
__device__ __forceinline__ float ld_c(const float* p) { return *p; }
__device__ __forceinline__ float ld_c(const uint16_t* p) { return __uint_as_float((uint32_t)(*p) << 16); }
__device__ __forceinline__ void st_c(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_c(uint16_t* p, float v) { *p = f32_to_bf16_rne(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {      // red: >= 33 floats of shared memory; all threads get the sum
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }

// The tensor-core GEMMs take an f32 activation as two bf16 halves, v = hi + lo (about 16 mantissa bits): written by the kernel
// that produces the activation, beside the f32 copy.  hi == nullptr: the exact path, nothing to write.
__device__ __forceinline__ void split_store(uint16_t* hi, uint16_t* lo, size_t i, float v) {
    if (hi == nullptr) return;
    const uint16_t h = f32_to_bf16_rne(v);
    hi[i] = h;
    lo[i] = f32_to_bf16_rne(v - __uint_as_float((uint32_t)h << 16));
}
static __global__ void ly_split_kernel(const float* __restrict__ x, size_t n, uint16_t* __restrict__ hi, uint16_t* __restrict__ lo) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) split_store(hi, lo, i, x[i]);
}
// V consecutive floats at once (V = 4: one 16-byte access; the address must be 16-byte aligned) and their hi | lo halves
template <int V>
__device__ __forceinline__ void ld_vec(const float* p, float (&o)[V]) {
    if constexpr (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w; }
    else {
#pragma unroll
        for (int i = 0; i < V; ++i) o[i] = p[i];
    }
}
template <int V>
__device__ __forceinline__ void st_vec(float* p, const float (&o)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
    else {
#pragma unroll
        for (int i = 0; i < V; ++i) p[i] = o[i];
    }
}
template <int V>
__device__ __forceinline__ void split_store_vec(uint16_t* hi, uint16_t* lo, size_t i, const float (&o)[V]) {
    if (hi == nullptr) return;
    uint16_t h[V], l[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
        h[k] = f32_to_bf16_rne(o[k]);
        l[k] = f32_to_bf16_rne(o[k] - __uint_as_float((uint32_t)h[k] << 16));
    }
    if constexpr (V == 4) {
        *reinterpret_cast<uint2*>(hi + i) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
        *reinterpret_cast<uint2*>(lo + i) = make_uint2((uint32_t)l[0] | ((uint32_t)l[1] << 16), (uint32_t)l[2] | ((uint32_t)l[3] << 16));
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) { hi[i + k] = h[k]; lo[i + k] = l[k]; }
    }
}
// out[i] = sum over the split-K slices of a tensor-core GEMM, in slice order
static __global__ void ly_sum_slices_kernel(const float* __restrict__ y, int nsl, size_t stride, size_t n, float* __restrict__ out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float t = 0.f;
        for (int k = 0; k < nsl; ++k) t += y[(size_t)k * stride + i];
        out[i] = t;
    }
}

// ---- embedding + first norm ------------------------------------------------------------------------------------------------
// A norm weight w scales by (1 + w), or by w itself when `plain`.
__device__ __forceinline__ float norm_scale(const float* __restrict__ w, int c, int plain) { return plain ? w[c] : 1.f + w[c]; }

// x[row] = embed[tok[row]] (times escale when that is not 0) (+ pos_tab[row_pos[row]], a learned position vector);  h[row] = x / sqrt(mean x^2 + eps) * scale(w).
// nw == nullptr (the first sublayer reads the stream itself): h is not written and the hi | lo halves are those of x.
// x0 (optional): a second copy of x, the first entry of the depth average's history.
static __global__ void ly_embed_norm_kernel(const uint16_t* __restrict__ embed, const int* __restrict__ tok, int W, const float* __restrict__ nw,
                                            float eps, int plain, const uint16_t* __restrict__ pos_tab, const int* __restrict__ row_pos,
                                            float escale, float* __restrict__ x, float* __restrict__ x0, float* __restrict__ h,
                                            uint16_t* __restrict__ hhi, uint16_t* __restrict__ hlo) {
    __shared__ float red[33];
    const int row = blockIdx.x;
    const uint16_t* e = embed + (size_t)tok[row] * W;
    const uint16_t* pe = pos_tab ? pos_tab + (size_t)row_pos[row] * W : nullptr;
    float* xr = x + (size_t)row * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = __uint_as_float((uint32_t)e[c] << 16);
        if (escale != 0.f) v *= escale;
        if (pe) v += __uint_as_float((uint32_t)pe[c] << 16);
        xr[c] = v;
        if (x0) x0[(size_t)row * W + c] = v;
        ss += v * v;
        if (nw == nullptr) split_store(hhi, hlo, (size_t)row * W + c, v);
    }
    if (nw == nullptr) return;
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    float* hr = h + (size_t)row * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c] * r * norm_scale(nw, c, plain);
        hr[c] = v;
        split_store(hhi, hlo, (size_t)row * W + c, v);
    }
}

// x[row] += norm(y[row] + yb; wb);  then, if wnext, h[row] = norm(x[row]; wnext); else, if split_x, the hi | lo halves of x[row]
// itself (the next sublayer reads the stream un-normed).  yb: optional bias of the projection that produced y.
static __global__ void ly_post_norm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ yb, const float* __restrict__ wb,
                                           const float* __restrict__ wnext, float eps, int W, int plain, int split_x, float* __restrict__ h,
                                           uint16_t* __restrict__ hhi, uint16_t* __restrict__ hlo) {
    __shared__ float red[33];
    const int row = blockIdx.x;
    const float* yr = y + (size_t)row * W;
    float* xr = x + (size_t)row * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = yr[c] + (yb ? yb[c] : 0.f);
        ss += v * v;
    }
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c] + (yr[c] + (yb ? yb[c] : 0.f)) * r * norm_scale(wb, c, plain);
        xr[c] = v;
        s2 += v * v;
        if (wnext == nullptr && split_x) split_store(hhi, hlo, (size_t)row * W + c, v);
    }
    if (wnext == nullptr) return;
    const float r2 = 1.f / sqrtf(block_sum(s2, red) / (float)W + eps);
    float* hr = h + (size_t)row * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c] * r2 * norm_scale(wnext, c, plain);
        hr[c] = v;
        split_store(hhi, hlo, (size_t)row * W + c, v);
    }
}

// A sublayer's result joins the stream un-normed:  x[row] += gate * v,  where
//   v = y[row], or with two mixers side by side (y2 != nullptr) v = (unit(y) * wa + unit(y2) * wb) / 2, unit(.) = . / sqrt(mean .^2 + eps);
//   gate = sigmoid(gz[row] + gb) per channel (gz == nullptr: 1).
// slot >= 0 (the layer's last sublayer, stacks with a depth average): hist[slot][row] = x[row], the layer's own result, and then
//   x[row] = sum_{j <= slot} dw[j] * hist[j][row]  (hist[0] = the embedding output), in ascending j.
// Then, if wnext, h[row] = norm(x[row]; wnext) with its hi | lo halves.
// One block per row; a thread takes V consecutive channels at a time (V = 4: 16-byte accesses, W a multiple of 4).
template <int V>
static __global__ void ly_join_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ y2, const float* __restrict__ wa,
                                      const float* __restrict__ wb, const float* __restrict__ gz, const float* __restrict__ gb,
                                      float* __restrict__ hist, size_t hist_stride, int slot, const float* __restrict__ dw,
                                      const float* __restrict__ wnext, float eps, int W, int plain, float* __restrict__ h,
                                      uint16_t* __restrict__ hhi, uint16_t* __restrict__ hlo) {
    __shared__ float red[33];
    const int row = blockIdx.x;
    const size_t rb = (size_t)row * W;
    const int step = blockDim.x * V;
    float ra = 1.f, rb2 = 1.f;
    if (y2 != nullptr) {
        float sa = 0.f, sb = 0.f;
        for (int c = threadIdx.x * V; c < W; c += step) {
            float p[V], q[V];
            ld_vec<V>(y + rb + c, p); ld_vec<V>(y2 + rb + c, q);
#pragma unroll
            for (int i = 0; i < V; ++i) { sa += p[i] * p[i]; sb += q[i] * q[i]; }
        }
        ra = 1.f / sqrtf(block_sum(sa, red) / (float)W + eps);
        rb2 = 1.f / sqrtf(block_sum(sb, red) / (float)W + eps);
    }
    float s2 = 0.f;
    for (int c = threadIdx.x * V; c < W; c += step) {
        float v[V], t[V];
        ld_vec<V>(y + rb + c, v);
        if (y2 != nullptr) {
            float q[V], fa[V], fb[V];
            ld_vec<V>(y2 + rb + c, q); ld_vec<V>(wa + c, fa); ld_vec<V>(wb + c, fb);
#pragma unroll
            for (int i = 0; i < V; ++i) v[i] = 0.5f * (v[i] * ra * fa[i] + q[i] * rb2 * fb[i]);
        }
        if (gz != nullptr) {
            float z[V], bz[V];
            ld_vec<V>(gz + rb + c, z); ld_vec<V>(gb + c, bz);
#pragma unroll
            for (int i = 0; i < V; ++i) v[i] *= sigmoidf_(z[i] + bz[i]);
        }
        ld_vec<V>(x + rb + c, t);
#pragma unroll
        for (int i = 0; i < V; ++i) t[i] += v[i];
        if (slot >= 0) {
            st_vec<V>(hist + (size_t)slot * hist_stride + rb + c, t);
            float acc[V];
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = 0.f;
            for (int j = 0; j < slot; ++j) {
                float o[V];
                ld_vec<V>(hist + (size_t)j * hist_stride + rb + c, o);
                const float dj = dw[j];
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = fmaf(dj, o[i], acc[i]);
            }
            const float ds = dw[slot];
#pragma unroll
            for (int i = 0; i < V; ++i) t[i] = fmaf(ds, t[i], acc[i]);
        }
        st_vec<V>(x + rb + c, t);
#pragma unroll
        for (int i = 0; i < V; ++i) s2 += t[i] * t[i];
    }
    if (wnext == nullptr) return;
    const float r2 = 1.f / sqrtf(block_sum(s2, red) / (float)W + eps);
    for (int c = threadIdx.x * V; c < W; c += step) {
        float t[V], wn[V];
        ld_vec<V>(x + rb + c, t); ld_vec<V>(wnext + c, wn);
#pragma unroll
        for (int i = 0; i < V; ++i) t[i] = t[i] * r2 * (plain ? wn[i] : 1.f + wn[i]);
        st_vec<V>(h + rb + c, t);
        split_store_vec<V>(hhi, hlo, rb + c, t);
    }
}

// The norm follows the sum:  x[row] <- unit(alpha x[row] + sa (y[row] + yb) + sb y2[row]) * w,  unit(v) = v / sqrt(mean v^2 + eps); y2 and
// yb are optional.  split_x: also the hi | lo halves of the new x (the next sublayer reads the stream itself).  One block per row, V
// consecutive channels per thread (V = 4: 16-byte accesses, W a multiple of 4); the summed row waits in shared memory ([W] floats)
// between the two passes.
template <int V>
static __global__ void ly_sum_norm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ yb, const float* __restrict__ y2,
                                          float alpha, float sa, float sb, const float* __restrict__ w, float eps, int W, int plain, int split_x,
                                          uint16_t* __restrict__ hhi, uint16_t* __restrict__ hlo) {
    extern __shared__ __align__(16) float srow[];
    __shared__ float red[33];
    const size_t rb = (size_t)blockIdx.x * W;
    const int step = blockDim.x * V;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < W; c += step) {
        float t[V], p[V];
        ld_vec<V>(x + rb + c, t); ld_vec<V>(y + rb + c, p);
        if (yb != nullptr) {
            float b[V];
            ld_vec<V>(yb + c, b);
#pragma unroll
            for (int i = 0; i < V; ++i) p[i] += b[i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) t[i] = fmaf(alpha, t[i], sa * p[i]);
        if (y2 != nullptr) {
            float q[V];
            ld_vec<V>(y2 + rb + c, q);
#pragma unroll
            for (int i = 0; i < V; ++i) t[i] = fmaf(sb, q[i], t[i]);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) ss += t[i] * t[i];
        st_vec<V>(srow + c, t);
    }
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    for (int c = threadIdx.x * V; c < W; c += step) {
        float t[V], wn[V];
        ld_vec<V>(srow + c, t); ld_vec<V>(w + c, wn);
#pragma unroll
        for (int i = 0; i < V; ++i) t[i] = t[i] * r * (plain ? wn[i] : 1.f + wn[i]);
        st_vec<V>(x + rb + c, t);
        if (split_x) split_store_vec<V>(hhi, hlo, rb + c, t);
    }
}

// logits <- cap tanh(logits / cap)
static __global__ void ly_softcap_kernel(float* __restrict__ z, size_t n, float cap) {
    const float inv = 1.f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) z[i] = cap * tanhf(z[i] * inv);
}

// hf[i] = norm(x[want[i]]; w): the rows that go on to the vocabulary projection
static __global__ void ly_final_norm_kernel(const float* __restrict__ x, const int* __restrict__ want, const float* __restrict__ w, float eps, int W,
                                            int plain, float* __restrict__ hf, uint16_t* __restrict__ hhi, uint16_t* __restrict__ hlo) {
    __shared__ float red[33];
    const float* xr = x + (size_t)want[blockIdx.x] * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ss += xr[c] * xr[c];
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    float* hr = hf + (size_t)blockIdx.x * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c] * r * norm_scale(w, c, plain);
        hr[c] = v;
        split_store(hhi, hlo, (size_t)blockIdx.x * W + c, v);
    }
}

// ---- exact GEMM: Y[p, n] = sum_k A[row(p), k] * W[n, k]   (A f32, W bf16 bit patterns, f32 FMA in ascending k) ----------------------
// Strided groups (blockIdx.z): group g uses A + g*a_gs, W + g*w_gs, Y + g*y_gs and the rows p in [grp_off[g], grp_off[g+1])
// (grp_off == nullptr: rows [0, R) for every group).  a_idx gathers A rows (row(p) = a_idx[p]).
struct LyGemm {
    const float* A; long long a_gs; int lda; const int* a_idx;
    const uint16_t* W; long long w_gs; int N, K;
    float* Y; long long y_gs; int ldy;
    const int* grp_off; int R;
};
constexpr int kLyBM = 64, kLyBN = 64, kLyBK = 16;

// Acc = double (the exact mode): every output is the correctly rounded f32 of its dot product, whatever K.
template <typename Acc>
static __global__ void __launch_bounds__(256) ly_gemm_kernel(LyGemm g) {
    __shared__ float As[kLyBK][kLyBM + 4];
    __shared__ float Ws[kLyBK][kLyBN + 4];
    const int grp = blockIdx.z;
    int p_lo = 0, p_hi = g.R;
    if (g.grp_off != nullptr) { p_lo = g.grp_off[grp]; p_hi = g.grp_off[grp + 1]; }
    const int p0 = p_lo + blockIdx.y * kLyBM;
    if (p0 >= p_hi) return;
    const int n0 = blockIdx.x * kLyBN;
    const float* A = g.A + (size_t)grp * g.a_gs;
    const uint16_t* Wm = g.W + (size_t)grp * g.w_gs;
    float* Y = g.Y + (size_t)grp * g.y_gs;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int lr = tid >> 2, lk = (tid & 3) * 4;            // loader: row / first k of this thread's 4 elements
    const int ap = p0 + lr;
    const float* arow = nullptr;
    if (ap < p_hi) arow = A + (size_t)(g.a_idx ? g.a_idx[ap] : ap) * g.lda;
    const uint16_t* wrow = (n0 + lr < g.N) ? Wm + (size_t)(n0 + lr) * g.K : nullptr;
    Acc acc[4][4] = {};
    for (int k0 = 0; k0 < g.K; k0 += kLyBK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            As[lk + i][lr] = (arow != nullptr && k < g.K) ? arow[k] : 0.f;
            Ws[lk + i][lr] = (wrow != nullptr && k < g.K) ? __uint_as_float((uint32_t)wrow[k] << 16) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kLyBK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fma((Acc)a[i], (Acc)b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = p0 + ty * 4 + i;
        if (p >= p_hi) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < g.N) Y[(size_t)p * g.ldy + n] = (float)acc[i][j];
        }
    }
}

// ---- gated linear attention ------------------------------------------------------------------------------------------------
struct GlaArgs {
    const float* proj; int ldp, off_q, off_k, off_v;
    const float* z;             // [T, H*D] decay pre-activation W_a2 (W_a1 h), without the bias
    const float* zb;            // [H*D] its bias
    float inv_tau;
    float* o;                   // [T, H*Dv]
    float* state;               // [slots][H][D][Dv]
    const int *seq_row0, *seq_slot, *seq_pos0;
    int H, D, Dv;
    float qscale;
};
constexpr int kGlaVS = 32, kGlaDG = 8;        // value columns per block, key-channel groups per block

// The recurrence itself, token by token: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_t * qscale).  One block per
// (sequence, head, 32 value columns): columns of S never interact, so the state is cut along vdim.  Thread (vcol, dg) keeps rows
// dg, dg + 8, ... of its column in registers.  The order of operations per token does not depend on how a prompt was cut.
template <int RPT>
static __global__ void __launch_bounds__(kGlaVS * kGlaDG) ly_gla_scan_kernel(GlaArgs a) {
    extern __shared__ float sm[];
    const int D = a.D, Dv = a.Dv;
    float* sq = sm;                     // [2][D]
    float* sk = sq + 2 * D;             // [2][D]
    float* sa = sk + 2 * D;             // [2][D]
    float* sv = sa + 2 * D;             // [2][32]
    float* red = sv + 2 * kGlaVS;       // [2][8][32]
    const int seq = blockIdx.x, hd = blockIdx.y, v0 = blockIdx.z * kGlaVS;
    const int tid = threadIdx.x, vc = tid & 31, dg = tid >> 5;
    const int r0 = a.seq_row0[seq], r1 = a.seq_row0[seq + 1];
    const bool vok = v0 + vc < Dv;
    float* st = a.state + (((size_t)a.seq_slot[seq] * a.H + hd) * D) * Dv + v0 + vc;
    float s[RPT];
    const bool fresh = a.seq_pos0[seq] == 0;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int d = dg + kGlaDG * i;
        s[i] = (!fresh && vok && d < D) ? st[(size_t)d * Dv] : 0.f;
    }
    // Software pipeline: the next token's q / k / z / v travel from global memory into registers while the current token is folded
    // into the state; they are written to the other shared-memory buffer afterwards.  One block barrier per token.
    const bool ld_d = tid < D, ld_v = tid < kGlaVS;      // D <= 256 = blockDim: a thread fetches at most one channel of each vector
    float rq = 0.f, rk = 0.f, rz = 0.f, rv = 0.f;
    auto fetch = [&](int row) {
        const float* pr = a.proj + (size_t)row * a.ldp;
        if (ld_d) {
            rq = pr[a.off_q + hd * D + tid];
            rk = pr[a.off_k + hd * D + tid];
            rz = a.z[(size_t)row * a.H * D + hd * D + tid];
        }
        if (ld_v) rv = (v0 + tid < Dv) ? pr[a.off_v + hd * Dv + v0 + tid] : 0.f;
    };
    const float zb = ld_d ? a.zb[hd * D + tid] : 0.f;
    auto stage = [&](int b) {
        if (ld_d) {
            sq[b * D + tid] = rq * a.qscale;
            sk[b * D + tid] = rk;
            // alpha = sigmoid(z)^(1/tau) = exp(log sigmoid(z) / tau),  log sigmoid(z) = -(max(-z, 0) + log1p(exp(-|z|)))
            const float z = rz + zb;
            sa[b * D + tid] = expf(-(fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)))) * a.inv_tau);
        }
        if (ld_v) sv[b * kGlaVS + tid] = rv;
    };
    auto finish = [&](int row, int b) {              // add the 8 partial sums of a token in a fixed order
        if (dg == 0 && vok) {
            const float* rp = red + b * kGlaDG * kGlaVS;
            float t = 0.f;
#pragma unroll
            for (int g = 0; g < kGlaDG; ++g) t += rp[g * kGlaVS + vc];
            a.o[(size_t)row * a.H * Dv + hd * Dv + v0 + vc] = t;
        }
    };
    if (r0 < r1) { fetch(r0); stage(0); }
    int b = 0;
    for (int row = r0; row < r1; ++row, b ^= 1) {
        if (row + 1 < r1) fetch(row + 1);
        __syncthreads();
        if (row > r0) finish(row - 1, b ^ 1);
        const float v = sv[b * kGlaVS + vc];
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int d = dg + kGlaDG * i;
            if (d < D) {
                s[i] = fmaf(s[i], sa[b * D + d], sk[b * D + d] * v);
                acc = fmaf(s[i], sq[b * D + d], acc);
            }
        }
        red[(b * kGlaDG + dg) * kGlaVS + vc] = acc;
        if (row + 1 < r1) stage(b ^ 1);
    }
    __syncthreads();
    if (r0 < r1) finish(r1 - 1, b ^ 1);
    if (vok) {
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int d = dg + kGlaDG * i;
            if (d < D) st[(size_t)d * Dv] = s[i];
        }
    }
}

// u[row, h, :] = o[row, h, :] / sqrt(mean o^2 + eps) * w[:] * silu(g[row, h, :])     (one warp per (row, head))
static __global__ void ly_gla_out_kernel(const float* __restrict__ o, const float* __restrict__ proj, int ldp, int off_g, const float* __restrict__ w,
                                         float eps, int T, int H, int Dv, float* __restrict__ u, uint16_t* __restrict__ uhi, uint16_t* __restrict__ ulo) {
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= T * H) return;
    const int row = item / H, hd = item % H;
    const float* op = o + (size_t)row * H * Dv + hd * Dv;
    float ss = 0.f;
    for (int c = lane; c < Dv; c += 32) ss += op[c] * op[c];
    const float r = 1.f / sqrtf(warp_sum(ss) / (float)Dv + eps);
    const float* gp = proj + (size_t)row * ldp + off_g + hd * Dv;
    float* up = u + (size_t)row * H * Dv + hd * Dv;
    for (int c = lane; c < Dv; c += 32) {
        const float g = gp[c];
        const float v = op[c] * r * w[c] * (g * sigmoidf_(g));
        up[c] = v;
        split_store(uhi, ulo, (size_t)row * H * Dv + hd * Dv + c, v);
    }
}

// ---- latent attention ------------------------------------------------------------------------------------------------------
struct LatentAppendArgs {
    float* proj; int ldp, off_q, off_dkv;       // off_dkv < 0: the layer reads another layer's cache (queries are still rotated)
    const float* dkv_norm; float eps;
    void* pool;                                  // [pages][64][C + R]
    const int* page_table; int pps;
    const int *row_seq, *row_pos, *seq_slot;
    const float *cosb, *sinb;                    // [max_seq][rdims / 2], already multiplied by the YaRN magnitude
    int H, D, R, C, rdims;
};
// Per row: the latent (RMS-normed, plain weight) and the rotated shared key part go into the row's cache page; the rotated part of
// every head's query is turned in place.  Pairs (2i, 2i+1) of the first rdims channels turn by pos * f_i; the rest pass through.
template <typename CT>
static __global__ void ly_latent_append_kernel(LatentAppendArgs a) {
    __shared__ float red[33];
    const int row = blockIdx.x, pos = a.row_pos[row];
    float* pr = a.proj + (size_t)row * a.ldp;
    const float* cs = a.cosb + (size_t)pos * (a.rdims / 2);
    const float* sn = a.sinb + (size_t)pos * (a.rdims / 2);
    for (int i = threadIdx.x; i < a.H * (a.rdims / 2); i += blockDim.x) {
        const int hd = i / (a.rdims / 2), pi = i % (a.rdims / 2);
        float* q = pr + a.off_q + hd * (a.D + a.R) + a.D + 2 * pi;
        const float u = q[0], v = q[1];
        q[0] = u * cs[pi] - v * sn[pi];
        q[1] = v * cs[pi] + u * sn[pi];
    }
    if (a.off_dkv < 0) return;
    const int slot = a.seq_slot[a.row_seq[row]];
    const int page = a.page_table[(size_t)slot * a.pps + pos / kKvPage];
    CT* dst = (CT*)a.pool + ((size_t)page * kKvPage + pos % kKvPage) * (a.C + a.R);
    const float* ckv = pr + a.off_dkv;
    float ss = 0.f;
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) ss += ckv[c] * ckv[c];
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)a.C + a.eps);
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) st_c(dst + c, ckv[c] * r * a.dkv_norm[c]);
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) {
        float val;
        if (i < a.rdims) {
            const int pi = i >> 1;
            const float u = ckv[a.C + 2 * pi], v = ckv[a.C + 2 * pi + 1];
            val = (i & 1) ? v * cs[pi] + u * sn[pi] : u * cs[pi] - v * sn[pi];
        } else {
            val = ckv[a.C + i];
        }
        st_c(dst + a.C + i, val);
    }
}

struct LatentAttnArgs {
    const float* qa;            // [T, H, C] queries with W_uk absorbed
    const float* proj; int ldp, off_q;          // rotated query part lives at proj[row, off_q + h (D + R) + D ...]
    const void* pool; const int* page_table; int pps;
    const int *row_seq, *row_pos, *seq_slot;
    float* ol;                  // [T, H, C] softmax-weighted sum of latents
    int H, D, R, C, window;
    float scale;
    int row_base;               // first row of this launch (blockIdx.x counts from it)
};
// CPL consecutive cache elements starting at channel c0 of a key row, as f32; channels >= C read as zero.  16-byte loads when the
// chunk is whole, inside the latent and aligned; single elements otherwise.
template <int CPL>
__device__ __forceinline__ void load_chunk(const float* kp, int c0, int C, float* out) {
    if (CPL % 4 == 0 && c0 + CPL <= C && (reinterpret_cast<uintptr_t>(kp + c0) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < CPL / 4; ++i) {
            const float4 v = reinterpret_cast<const float4*>(kp + c0)[i];
            out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < CPL; ++i) out[i] = c0 + i < C ? kp[c0 + i] : 0.f;
    }
}
template <int CPL>
__device__ __forceinline__ void load_chunk(const uint16_t* kp, int c0, int C, float* out) {
    if (CPL % 8 == 0 && c0 + CPL <= C && (reinterpret_cast<uintptr_t>(kp + c0) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < CPL / 8; ++i) {
            const uint4 v = reinterpret_cast<const uint4*>(kp + c0)[i];
            out[8 * i] = bf16lo(v.x); out[8 * i + 1] = bf16hi(v.x); out[8 * i + 2] = bf16lo(v.y); out[8 * i + 3] = bf16hi(v.y);
            out[8 * i + 4] = bf16lo(v.z); out[8 * i + 5] = bf16hi(v.z); out[8 * i + 6] = bf16lo(v.w); out[8 * i + 7] = bf16hi(v.w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < CPL; ++i) out[i] = c0 + i < C ? ld_c(kp + c0 + i) : 0.f;
    }
}

constexpr int kLatWarps = 8;
// One block per (row, head).  score_j = (q~ . c_j + q_rot . k_rot_j) * scale over the keys j the window admits (0 <= pos - j <
// window), softmax in f32, out = sum_j p_j c_j.  Warp w of the eight folds keys j0 + w, j0 + w + 8, ... into an online softmax (lanes own
// channels); the eight partial results are merged at the end.  Which warp takes which key depends on the position alone.
template <typename CT, int CPL>
static __global__ void __launch_bounds__(kLatWarps * 32) ly_latent_attn_kernel(LatentAttnArgs a) {
    extern __shared__ float sm[];               // [kLatWarps][C] accumulators, then [kLatWarps][2] (max, sum)
    constexpr int RPL = 4;                      // rotated channels per lane (R <= 128)
    const int row = a.row_base + blockIdx.x, hd = blockIdx.y, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int C = a.C, R = a.R, E = C + R;
    const int pos = a.row_pos[row], slot = a.seq_slot[a.row_seq[row]];
    const int j0 = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    float q[CPL], qr[RPL], acc[CPL];
    const float* qap = a.qa + ((size_t)row * a.H + hd) * C;
    const float* qrp = a.proj + (size_t)row * a.ldp + a.off_q + hd * (a.D + R) + a.D;
#pragma unroll
    for (int i = 0; i < CPL; ++i) { const int c = lane * CPL + i; q[i] = c < C ? qap[c] : 0.f; acc[i] = 0.f; }      // a lane owns CPL consecutive channels
#pragma unroll
    for (int i = 0; i < RPL; ++i) { const int c = lane * RPL + i; qr[i] = c < R ? qrp[c] : 0.f; }
    float m = -INFINITY, l = 0.f;
    const int* pt = a.page_table + (size_t)slot * a.pps;
    constexpr int KU = 2;                       // keys in flight per warp: their loads and reductions overlap, the folds stay in key order
    for (int j = j0 + wid; j <= pos; j += kLatWarps * KU) {
        float lat[KU][CPL], dot[KU];
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int jj = j + u * kLatWarps;
            dot[u] = 0.f;
            if (jj <= pos) {
                const CT* kp = (const CT*)a.pool + ((size_t)pt[jj / kKvPage] * kKvPage + jj % kKvPage) * E;
#pragma unroll
                load_chunk<CPL>(kp, lane * CPL, C, lat[u]);
                float kr[RPL];
                load_chunk<RPL>(kp + C, lane * RPL, R, kr);
#pragma unroll
                for (int i = 0; i < CPL; ++i) dot[u] = fmaf(q[i], lat[u][i], dot[u]);
#pragma unroll
                for (int i = 0; i < RPL; ++i) dot[u] = fmaf(qr[i], kr[i], dot[u]);
            } else {
#pragma unroll
                for (int i = 0; i < CPL; ++i) lat[u][i] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < KU; ++u) dot[u] = warp_sum(dot[u]) * a.scale;
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            if (j + u * kLatWarps > pos) break;
            const float sc = dot[u];
            const float mn = fmaxf(m, sc), corr = expf(m - mn), p = expf(sc - mn);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < CPL; ++i) acc[i] = acc[i] * corr + p * lat[u][i];
            m = mn;
        }
    }
    float* sacc = sm;
    float* sml = sm + kLatWarps * C;
#pragma unroll
    for (int i = 0; i < CPL; ++i) { const int c = lane * CPL + i; if (c < C) sacc[wid * C + c] = acc[i]; }
    if (lane == 0) { sml[2 * wid] = m; sml[2 * wid + 1] = l; }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kLatWarps; ++w) M = fmaxf(M, sml[2 * w]);
    float f[kLatWarps], Lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kLatWarps; ++w) { f[w] = expf(sml[2 * w] - M); Lsum += sml[2 * w + 1] * f[w]; }
    const float inv = 1.f / Lsum;
    float* op = a.ol + ((size_t)row * a.H + hd) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kLatWarps; ++w) t += sacc[w * C + c] * f[w];
        op[c] = t * inv;
    }
}

// ---- latent attention for long portions on the tensor-core GEMM (serving precision) ---------------------------------------------
// A block of consecutive query rows of ONE sequence and the keys its window can reach [k_lo, k_lo + nk):
//   S = Q~ . Kc^T (one GEMM: rows = (token, head) pairs -- every head of a token meets the same latent keys),
//   P = masked softmax(S) in f32,   O = P . Kc[:, :C] (a second GEMM against the transposed latents).
// Kc [nkp, Ep]: the keys' cache rows (latent | rotated part | zero padding), KcT [C, nkp]: the latents transposed; padding is
// zero so that masked probabilities (exact zeros) meet finite values.
static __global__ void ly_attn_gather_keys_kernel(const uint16_t* __restrict__ pool, const int* __restrict__ page_row, int k_lo, int nk, int nkp, int C,
                                                  int E, int Ep, uint16_t* __restrict__ kc, uint16_t* __restrict__ kct) {
    const int r = blockIdx.x;
    const uint16_t* src = nullptr;
    if (r < nk) {
        const int j = k_lo + r;
        src = pool + ((size_t)page_row[j / kKvPage] * kKvPage + j % kKvPage) * E;
    }
    for (int c = threadIdx.x; c < Ep; c += blockDim.x) {
        const uint16_t v = (src != nullptr && c < E) ? src[c] : (uint16_t)0;
        kc[(size_t)r * Ep + c] = v;
        if (c < C) kct[(size_t)c * nkp + r] = v;
    }
}
// Q operand rows (token, head): [q~ * scale | rotated query part * scale | 0] as hi | lo halves
static __global__ void ly_attn_build_q_kernel(const float* __restrict__ qa, const float* __restrict__ proj, int ldp, int off_q, int row0, int H, int D,
                                              int R, int C, int Ep, float scale, uint16_t* __restrict__ qhi, uint16_t* __restrict__ qlo) {
    const int t = blockIdx.x, hd = blockIdx.y, row = row0 + t;
    const float* qap = qa + ((size_t)row * H + hd) * C;
    const float* qrp = proj + (size_t)row * ldp + off_q + hd * (D + R) + D;
    const size_t base = ((size_t)t * H + hd) * Ep;
    for (int c = threadIdx.x; c < Ep; c += blockDim.x) {
        const float v = c < C ? qap[c] * scale : (c < C + R ? qrp[c - C] * scale : 0.f);
        split_store(qhi, qlo, base + c, v);
    }
}
// Which keys position `pos` reads: with lo_c the start of its chunk (0 without chunks) and lo_w the start of its window (0 without one),
// the contiguous range [j0, pos], j0 = max(lo_w, lo_c), and before it the kept first keys [s_lo, s_hi) = [lo_c, min(keep_first, j0))
// (empty unless a window is set and s_lo < s_hi).
struct KeySpan { int j0, s_lo, s_hi; };
__device__ __forceinline__ KeySpan key_span(int pos, int window, int keep_first, int chunk) {
    const int lo_c = chunk > 0 ? pos / chunk * chunk : 0;
    const int lo_w = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    KeySpan k;
    k.j0 = max(lo_w, lo_c);
    k.s_lo = lo_c;
    k.s_hi = window > 0 ? max(lo_c, min(keep_first, k.j0)) : lo_c;
    return k;
}

// P[r, col] = softmax over the keys the row's position admits (key_span), zero elsewhere; row r belongs to token r / H of the block.
// Columns: the first n_first hold keys 0 .. n_first - 1 (kept first keys that lie before k_lo), column n_first + i holds key k_lo + i,
// i < nk.  softcap > 0: scores pass softcap * tanh(s / softcap) first; sink: the denominator gets exp(sinkv[r % H]) more (exp(0) when
// sinkv is nullptr).  The (capped) scores of the row are kept in shared memory after the first pass when `keep` floats of it were
// given to the launch and the row fits (a thread meets the same columns in every pass, so it reads back what it wrote itself).
static __global__ void ly_attn_softmax_kernel(const float* __restrict__ S, const int* __restrict__ row_pos, int row0, int H, int k_lo, int n_first, int nk,
                                              int nkp, int window, int keep_first, int chunk, float softcap, int sink, const float* __restrict__ sinkv,
                                              int keep, uint16_t* __restrict__ phi, uint16_t* __restrict__ plo) {
    extern __shared__ float srow[];
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const int pos = row_pos[row0 + (int)(r / H)];
    const KeySpan ks = key_span(pos, window, keep_first, chunk);
    // visible columns: [a_lo, a_hi) of the first part; of [b_lo, c_hi) in the main part those whose key passes `vis`
    const int a_lo = min(ks.s_lo, n_first), a_hi = min(ks.s_hi, n_first), na = a_hi - a_lo;
    const int first_main = ks.s_hi > max(ks.s_lo, k_lo) ? max(ks.s_lo, k_lo) : ks.j0;
    const int b_lo = n_first + max(first_main - k_lo, 0), c_hi = n_first + min(nk, pos - k_lo + 1);
    auto vis = [&](int c) { const int j = k_lo + c - n_first; return j >= ks.j0 || (j >= ks.s_lo && j < ks.s_hi); };
    const float* sr = S + r * nkp;
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
    const int nvis = na + max(c_hi - b_lo, 0);
    const bool kept = nvis <= keep;
    const float sv = sink ? (sinkv ? sinkv[r % H] : 0.f) : 0.f;
    auto score = [&](int c) { const float v = sr[c]; return softcap > 0.f ? softcap * tanhf(v * inv_cap) : v; };
    float m = sink ? sv : -INFINITY;
    for (int i = threadIdx.x; i < nvis; i += blockDim.x) {
        const int c = i < na ? a_lo + i : b_lo + (i - na);
        const float v = (i < na || vis(c)) ? score(c) : -INFINITY;
        if (kept) srow[i] = v;
        m = fmaxf(m, v);
    }
    m = warp_max(m);
    {
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
        __syncthreads();
        if (lane == 0) red[wid] = m;
        __syncthreads();
        float t = lane < nw ? red[lane] : -INFINITY;
        m = warp_max(t);
    }
    float sum = 0.f;
    for (int i = threadIdx.x; i < nvis; i += blockDim.x) {
        const int c = i < na ? a_lo + i : b_lo + (i - na);
        const float v = kept ? srow[i] : ((i < na || vis(c)) ? score(c) : -INFINITY);
        const float e = v == -INFINITY ? 0.f : expf(v - m);
        if (kept) srow[i] = e;
        sum += e;
    }
    const float inv = 1.f / (block_sum(sum, red) + (sink ? expf(sv - m) : 0.f));
    for (int c = threadIdx.x; c < nkp; c += blockDim.x) {
        float p = 0.f;
        int i = -1;
        if (c >= a_lo && c < a_hi) i = c - a_lo;
        else if (c >= b_lo && c < c_hi && c >= n_first && vis(c)) i = na + (c - b_lo);
        if (i >= 0) p = (kept ? srow[i] : expf(score(c) - m)) * inv;
        split_store(phi, plo, r * nkp + c, p);
    }
}

// ---- grouped-query attention over a paged key | value cache ---------------------------------------------------------------------
// Cache row of a token: [kv_heads][dim] keys (normed, rotated) then [kv_heads][vdim] values.
struct AttnPrepArgs {
    float* proj; int ldp, off_q, off_k, off_v;  // off_k < 0: the layer reads another layer's cache (queries are still prepared)
    const float *qnorm, *knorm; float eps;       // [dim] each ([H * dim], [G * dim] when `whole`)
    void* pool; const int* page_table; int pps;
    const int *row_seq, *row_pos, *seq_slot;
    const float *cosb, *sinb;                    // [max_seq][rdims / 2], already multiplied by the YaRN magnitude
    int H, G, D, Dv, rdims, halves;
    const float *bq, *bk, *bv;                   // projection biases [H * dim], [G * dim], [G * vdim] (nullptr: none)
    int whole;                                   // 1: q (and k) are normed over all heads' channels at once
};
// Per row: every query head and (when the layer owns its cache) every key head is RMS-normed over dim with a weight shared by the
// heads (qnorm == nullptr: they are used as projected), then its first rdims channels are turned by the row's position: pairs (i, i + rdims/2) when `halves`, else (2i, 2i+1).
// Queries are rewritten in place, keys and values go to the row's cache page.  grid (rows, head chunks): the warps of a row's blocks
// take the heads in turn.  Biases, when the projections have them, are added as the values are read; with `whole` the mean square is
// taken over all heads of q (of k) before any head is rewritten (one block per row then: gridDim.y = 1) and the weight is indexed by
// the channel inside the whole projection.
template <typename CT>
static __global__ void __launch_bounds__(256) ly_attn_prep_kernel(AttnPrepArgs a) {
    extern __shared__ float sm[];               // [warps][D]
    __shared__ float red[33];
    const int row = blockIdx.x, pos = a.row_pos[row], lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float* pr = a.proj + (size_t)row * a.ldp;
    const bool own = a.off_k >= 0;
    float rq = 0.f, rk = 0.f;
    if (a.whole && a.qnorm != nullptr) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < a.H * a.D; c += blockDim.x) { const float v = pr[a.off_q + c] + (a.bq ? a.bq[c] : 0.f); ss += v * v; }
        rq = 1.f / sqrtf(block_sum(ss, red) / (float)(a.H * a.D) + a.eps);
        if (own) {
            ss = 0.f;
            for (int c = threadIdx.x; c < a.G * a.D; c += blockDim.x) { const float v = pr[a.off_k + c] + (a.bk ? a.bk[c] : 0.f); ss += v * v; }
            rk = 1.f / sqrtf(block_sum(ss, red) / (float)(a.G * a.D) + a.eps);
        }
    }
    const int half = a.rdims / 2;
    const float* cs = a.cosb + (size_t)pos * half;
    const float* sn = a.sinb + (size_t)pos * half;
    float* buf = sm + wid * a.D;
    CT* dst = nullptr;
    if (own) {
        const int slot = a.seq_slot[a.row_seq[row]];
        const int page = a.page_table[(size_t)slot * a.pps + pos / kKvPage];
        dst = (CT*)a.pool + ((size_t)page * kKvPage + pos % kKvPage) * ((size_t)a.G * (a.D + a.Dv));
    }
    const int items = a.H + (own ? a.G : 0);
    for (int it = blockIdx.y * nw + wid; it < items; it += gridDim.y * nw) {
        const bool isq = it < a.H;
        const int hd = isq ? it : it - a.H;
        float* src = isq ? pr + a.off_q + hd * a.D : pr + a.off_k + hd * a.D;
        const float* bias = isq ? a.bq : a.bk;
        if (bias != nullptr) bias += (size_t)hd * a.D;
        const float* w = isq ? a.qnorm : a.knorm;
        for (int c = lane; c < a.D; c += 32) buf[c] = src[c] + (bias ? bias[c] : 0.f);
        __syncwarp();
        if (w != nullptr) {
            float r;
            if (a.whole) {
                r = isq ? rq : rk;
                w += (size_t)hd * a.D;
            } else {
                float ss = 0.f;
                for (int c = lane; c < a.D; c += 32) ss += buf[c] * buf[c];
                r = 1.f / sqrtf(warp_sum(ss) / (float)a.D + a.eps);
            }
            for (int c = lane; c < a.D; c += 32) buf[c] = buf[c] * r * w[c];
            __syncwarp();
        }
        for (int c = lane; c < a.D; c += 32) {
            float val = buf[c];
            if (c < a.rdims) {
                int pi, second;
                if (a.halves) { second = c >= half; pi = second ? c - half : c; }
                else { second = c & 1; pi = c >> 1; }
                const int cu = a.halves ? pi : 2 * pi, cv = a.halves ? pi + half : 2 * pi + 1;
                const float u = buf[cu], v = buf[cv];
                val = second ? v * cs[pi] + u * sn[pi] : u * cs[pi] - v * sn[pi];
            }
            if (isq) src[c] = val; else st_c(dst + (size_t)hd * a.D + c, val);
        }
        __syncwarp();
    }
    if (own && blockIdx.y == 0) {
        const float* v = pr + a.off_v;
        CT* vd = dst + (size_t)a.G * a.D;
        for (int c = threadIdx.x; c < a.G * a.Dv; c += blockDim.x) st_c(vd + c, v[c] + (a.bv ? a.bv[c] : 0.f));
    }
}

struct GqaAttnArgs {
    const float* proj; int ldp, off_q;          // prepared queries at proj[row, off_q + h * D ...]
    const void* pool; const int* page_table; int pps;
    const int *row_seq, *row_pos, *seq_slot;
    float* out;                 // [T, H * Dv]
    uint16_t *ohi, *olo;        // its hi | lo halves (nullptr: not wanted)
    int H, G, D, Dv, window;
    float scale, softcap;       // softcap 0 = scores are used as they are
    int sink;                   // != 0: the denominator gets exp(sinkv[head]) more (exp(0) when sinkv is nullptr)
    int row_base;
    float* part;                // key splits (gridDim.z > 1): [T][H][splits][2 + Dv] partial (max, sum, weighted values)
    int keep_first, chunk;      // masks beside the window (see key_span)
    const float* sinkv;         // [H] or nullptr
};
constexpr int kGqaWarps = 8;
// One block per (row, RB query heads of one key/value head, key split).  score_j = cap(q . k_j * scale) over the keys the position
// admits (key_span: causal, window with kept first keys, chunk), softmax in f32 with the optional sink, out = sum_j p_j v_j.  The
// 8 x splits warps of a (row, head group) take the visible keys round-robin in ascending order: warp v folds the v-th, (v + 8 splits)-th,
// ... visible key into an online softmax per head (lanes own
// CPL consecutive channels of the key and of the value; a key and its value are loaded once for the RB heads).  Partial results
// are merged in warp order; with one split the block writes the output itself (which warp takes which key then depends on the
// position alone), otherwise ly_gqa_merge_kernel folds the splits in order.
template <typename CT, int CPL, int RB>
static __global__ void __launch_bounds__(kGqaWarps * 32) ly_gqa_attn_kernel(GqaAttnArgs a) {
    extern __shared__ float sm[];               // [warps][RB][Dv] accumulators, then [warps][RB][2] (max, sum)
    const int row = a.row_base + blockIdx.x, hd0 = blockIdx.y * RB, split = blockIdx.z, S = gridDim.z;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int D = a.D, Dv = a.Dv, g = hd0 / (a.H / a.G);
    const size_t E = (size_t)a.G * (D + Dv);
    const int pos = a.row_pos[row], slot = a.seq_slot[a.row_seq[row]];
    const KeySpan ks = key_span(pos, a.window, a.keep_first, a.chunk);
    const int n_st = ks.s_hi - ks.s_lo, n_vis = n_st + pos - ks.j0 + 1;        // kept first keys, then the contiguous range
    float q[RB][CPL], acc[RB][CPL], m[RB], l[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
        const float* qp = a.proj + (size_t)row * a.ldp + a.off_q + (size_t)(hd0 + r) * D;
#pragma unroll
        for (int i = 0; i < CPL; ++i) { const int c = lane * CPL + i; q[r][i] = c < D ? qp[c] * a.scale : 0.f; acc[r][i] = 0.f; }
        m[r] = -INFINITY; l[r] = 0.f;
    }
    const int* pt = a.page_table + (size_t)slot * a.pps;
    const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
    constexpr int KU = 2;
    const int stride = kGqaWarps * S;
    for (int j = split * kGqaWarps + wid; j < n_vis; j += stride * KU) {
        float val[KU][CPL], dot[KU][RB];
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int ji = j + u * stride, jj = ji < n_st ? ks.s_lo + ji : ks.j0 + (ji - n_st);
#pragma unroll
            for (int r = 0; r < RB; ++r) dot[u][r] = 0.f;
            if (ji < n_vis) {
                const CT* kp = (const CT*)a.pool + ((size_t)pt[jj / kKvPage] * kKvPage + jj % kKvPage) * E;
                float kk[CPL];
                load_chunk<CPL>(kp + (size_t)g * D, lane * CPL, D, kk);
                load_chunk<CPL>(kp + (size_t)a.G * D + (size_t)g * Dv, lane * CPL, Dv, val[u]);
#pragma unroll
                for (int r = 0; r < RB; ++r)
#pragma unroll
                    for (int i = 0; i < CPL; ++i) dot[u][r] = fmaf(q[r][i], kk[i], dot[u][r]);
            } else {
#pragma unroll
                for (int i = 0; i < CPL; ++i) val[u][i] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < KU; ++u)
#pragma unroll
            for (int r = 0; r < RB; ++r) dot[u][r] = warp_sum(dot[u][r]);
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            if (j + u * stride >= n_vis) break;
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                float sc = dot[u][r];
                if (a.softcap > 0.f) sc = a.softcap * tanhf(sc * inv_cap);
                const float mn = fmaxf(m[r], sc), corr = expf(m[r] - mn), p = expf(sc - mn);
                l[r] = l[r] * corr + p;
#pragma unroll
                for (int i = 0; i < CPL; ++i) acc[r][i] = acc[r][i] * corr + p * val[u][i];
                m[r] = mn;
            }
        }
    }
    float* sacc = sm;
    float* sml = sm + kGqaWarps * RB * Dv;
#pragma unroll
    for (int r = 0; r < RB; ++r) {
#pragma unroll
        for (int i = 0; i < CPL; ++i) { const int c = lane * CPL + i; if (c < Dv) sacc[(wid * RB + r) * Dv + c] = acc[r][i]; }
        if (lane == 0) { sml[(wid * RB + r) * 2] = m[r]; sml[(wid * RB + r) * 2 + 1] = l[r]; }
    }
    __syncthreads();
    for (int r = 0; r < RB; ++r) {
        const float sv = a.sinkv ? a.sinkv[hd0 + r] : 0.f;
        float M = (S == 1 && a.sink) ? sv : -INFINITY;
#pragma unroll
        for (int w = 0; w < kGqaWarps; ++w) M = fmaxf(M, sml[(w * RB + r) * 2]);
        float f[kGqaWarps], Lsum = (S == 1 && a.sink) ? expf(sv - M) : 0.f;
#pragma unroll
        for (int w = 0; w < kGqaWarps; ++w) {
            const float mw = sml[(w * RB + r) * 2];
            f[w] = mw == -INFINITY ? 0.f : expf(mw - M);       // a warp (or, with splits, a whole block) may have met no key
            Lsum += sml[(w * RB + r) * 2 + 1] * f[w];
        }
        if (S == 1) {
            const float inv = 1.f / Lsum;
            const size_t ob = ((size_t)row * a.H + hd0 + r) * Dv;
            for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < kGqaWarps; ++w) t += sacc[(w * RB + r) * Dv + c] * f[w];
                t *= inv;
                a.out[ob + c] = t;
                split_store(a.ohi, a.olo, ob + c, t);
            }
        } else {
            float* pp = a.part + (((size_t)blockIdx.x * a.H + hd0 + r) * S + split) * (Dv + 2);     // indexed by the row inside the launch
            if (threadIdx.x == 0) { pp[0] = M; pp[1] = Lsum; }
            for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < kGqaWarps; ++w) t += sacc[(w * RB + r) * Dv + c] * f[w];
                pp[2 + c] = t;
            }
        }
    }
}
// Folds the key splits of ly_gqa_attn_kernel in split order (and the sink): one block per (row, head).
static __global__ void ly_gqa_merge_kernel(const float* __restrict__ part, int S, int H, int Dv, int sink, const float* __restrict__ sinkv, int row_base,
                                           float* __restrict__ out, uint16_t* __restrict__ ohi, uint16_t* __restrict__ olo) {
    const int row = row_base + blockIdx.x, hd = blockIdx.y;
    const float* pp = part + ((size_t)blockIdx.x * H + hd) * S * (Dv + 2);
    const float sv = sinkv ? sinkv[hd] : 0.f;
    float M = sink ? sv : -INFINITY;
    for (int s = 0; s < S; ++s) M = fmaxf(M, pp[(size_t)s * (Dv + 2)]);
    float L = sink ? expf(sv - M) : 0.f;
    for (int s = 0; s < S; ++s) {
        const float ms = pp[(size_t)s * (Dv + 2)];
        L += ms == -INFINITY ? 0.f : pp[(size_t)s * (Dv + 2) + 1] * expf(ms - M);
    }
    const float inv = 1.f / L;
    const size_t ob = ((size_t)row * H + hd) * Dv;
    for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
        float t = 0.f;
        for (int s = 0; s < S; ++s) {
            const float ms = pp[(size_t)s * (Dv + 2)];
            if (ms != -INFINITY) t += pp[(size_t)s * (Dv + 2) + 2 + c] * expf(ms - M);
        }
        t *= inv;
        out[ob + c] = t;
        split_store(ohi, olo, ob + c, t);
    }
}

// ---- grouped-query attention of long portions on the tensor-core GEMM (serving precision) ---------------------------------------
// Per block of consecutive query rows of ONE sequence and per key/value head g: the keys the block can reach are gathered once
// (Kc [nkp, Dp], zero padded) with the values transposed (Vt [Dv, nkp]); the rows of the score GEMM are (token, query head of
// the group) pairs -- all of them meet the same keys --, S = Q . Kc^T, P = masked softmax(S) (cap, sink), O = P . V.
// Rows r < n_first hold keys 0 .. n_first - 1 (kept first keys before k_lo), rows n_first + i key k_lo + i, i < nk.
static __global__ void ly_gqa_gather_kv_kernel(const uint16_t* __restrict__ pool, const int* __restrict__ page_row, int k_lo, int n_first, int nk, int nkp,
                                               int E, int koff, int D, int Dp, int voff, int Dv, uint16_t* __restrict__ kc, uint16_t* __restrict__ vt) {
    const int r = blockIdx.x;
    const uint16_t* src = nullptr;
    if (r < n_first + nk) {
        const int j = r < n_first ? r : k_lo + (r - n_first);
        src = pool + ((size_t)page_row[j / kKvPage] * kKvPage + j % kKvPage) * E;
    }
    for (int c = threadIdx.x; c < Dp; c += blockDim.x) kc[(size_t)r * Dp + c] = (src != nullptr && c < D) ? src[koff + c] : (uint16_t)0;
    for (int c = threadIdx.x; c < Dv; c += blockDim.x) vt[(size_t)c * nkp + r] = src != nullptr ? src[voff + c] : (uint16_t)0;
}
// Q operand rows (token t, head hq of group g): the prepared query times `scale`, zero padded to Dp, as hi | lo halves.  grid (nq, rep)
static __global__ void ly_gqa_build_q_kernel(const float* __restrict__ proj, int ldp, int off_q, int row0, int rep, int g, int D, int Dp, float scale,
                                             uint16_t* __restrict__ qhi, uint16_t* __restrict__ qlo) {
    const int t = blockIdx.x, hq = blockIdx.y;
    const float* qp = proj + (size_t)(row0 + t) * ldp + off_q + (size_t)(g * rep + hq) * D;
    const size_t base = ((size_t)t * rep + hq) * Dp;
    for (int c = threadIdx.x; c < Dp; c += blockDim.x) split_store(qhi, qlo, base + c, c < D ? qp[c] * scale : 0.f);
}
// o [G][nq * rep][Dv] (the value GEMMs' outputs, one slab per key/value head) -> u[row0 + t, (g rep + hq) Dv + c] and its hi | lo halves
static __global__ void ly_gqa_scatter_kernel(const float* __restrict__ o, int nq, int G, int rep, int Dv, int row0, float* __restrict__ u,
                                             uint16_t* __restrict__ uhi, uint16_t* __restrict__ ulo) {
    const size_t total = (size_t)nq * G * rep * Dv;
    const int H = G * rep;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % Dv);
        const int hd = (int)((i / Dv) % H), t = (int)(i / ((size_t)Dv * H));
        const int g = hd / rep, hq = hd % rep;
        const float v = o[(((size_t)g * nq + t) * rep + hq) * Dv + c];
        const size_t dst = ((size_t)(row0 + t) * H + hd) * Dv + c;
        u[dst] = v;
        split_store(uhi, ulo, dst, v);
    }
}

// ---- recurrent mixers with a short causal convolution (Mamba-2, gated delta rule) --------------------------------------------------
__device__ __forceinline__ float softplusf_(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float siluf_(float z) { return z * sigmoidf_(z); }

constexpr int kMaxTaps = 16;
struct ConvArgs {
    const float* proj; int ldp, off;            // the convolved columns are proj[row, off .. off + ch)
    const float *w, *b;                         // [ch, taps], [ch] or nullptr
    float* state;                               // [slots][taps - 1][ch]: the inputs of the taps - 1 positions before the step, oldest first
    const int *row_seq, *row_pos, *seq_row0, *seq_slot, *seq_pos0;
    int ch, taps;
    float* cv;                                  // [T, ch]: silu(conv)
};
// Input of channel c at position p - back of the row's sequence: a row of this step, the slot's carried inputs, or zero before the start.
__device__ __forceinline__ float conv_input(const ConvArgs& a, int row, int row0, int pos, int pos0, int slot, int back, int c) {
    if (row - back >= row0) return a.proj[(size_t)(row - back) * a.ldp + a.off + c];
    const int p = pos - back;
    if (p < 0) return 0.f;
    return a.state[((size_t)slot * (a.taps - 1) + (p - pos0 + a.taps - 1)) * a.ch + c];
}
__device__ __forceinline__ float conv_silu(const ConvArgs& a, int row, int row0, int pos, int pos0, int slot, int c) {
    float t = a.b ? a.b[c] : 0.f;
    for (int k = 0; k < a.taps; ++k) t = fmaf(a.w[(size_t)c * a.taps + k], conv_input(a, row, row0, pos, pos0, slot, a.taps - 1 - k, c), t);
    return siluf_(t);
}
// After the rows of a step were convolved: the slot keeps the last taps - 1 inputs of each sequence.  grid (sequences, channel blocks).
static __global__ void ly_conv_state_kernel(ConvArgs a) {
    const int seq = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.ch) return;
    const int r0 = a.seq_row0[seq], n = a.seq_row0[seq + 1] - r0, pos0 = a.seq_pos0[seq], slot = a.seq_slot[seq];
    float keep[kMaxTaps];
    const int last_row = r0 + n - 1, last_pos = pos0 + n - 1;
    for (int i = 0; i < a.taps - 1; ++i) keep[i] = conv_input(a, last_row, r0, last_pos, pos0, slot, a.taps - 2 - i, c);
    for (int i = 0; i < a.taps - 1; ++i) a.state[((size_t)slot * (a.taps - 1) + i) * a.ch + c] = keep[i];
}

// Token shift in front of a mixer: out[row, c] = in[row, c] + (prev - in[row, c]) * mu[c], prev = the same channel of the sequence's
// previous position (a row of this step, the slot's carried row -- ConvArgs with taps = 2 --, or zero at position 0), with the hi | lo
// halves.  grid (rows, channel blocks of 128 x V); V = 4: 16-byte accesses (ch, ldp, off multiples of 4).
template <int V>
static __global__ void __launch_bounds__(128) ly_token_shift_kernel(ConvArgs a, const float* __restrict__ mu, float* __restrict__ out,
                                                                      uint16_t* __restrict__ ohi, uint16_t* __restrict__ olo) {
    const int row = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= a.ch) return;
    const int seq = a.row_seq[row], pos = a.row_pos[row];
    float cur[V], prev[V], m[V];
    ld_vec<V>(a.proj + (size_t)row * a.ldp + a.off + c, cur);
    ld_vec<V>(mu + c, m);
    if (row - 1 >= a.seq_row0[seq]) ld_vec<V>(a.proj + (size_t)(row - 1) * a.ldp + a.off + c, prev);
    else if (pos > 0) ld_vec<V>(a.state + (size_t)a.seq_slot[seq] * a.ch + c, prev);
    else {
#pragma unroll
        for (int i = 0; i < V; ++i) prev[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) cur[i] = cur[i] + (prev[i] - cur[i]) * m[i];
    st_vec<V>(out + (size_t)row * a.ch + c, cur);
    split_store_vec<V>(ohi, olo, (size_t)row * a.ch + c, cur);
}

// Lightning attention, per row: q | k | v <- silu(projection) (the columns proj[row, off .. off + ch) -> cv[row, :]); per head
// ab[row, h] = (decay[h], 1): the scan's fixed fade and a write strength of one.  grid (rows, channel chunks of `chunk`).
static __global__ void ly_lightning_prep_kernel(const float* __restrict__ proj, int ldp, int off, int ch, int chunk, const float* __restrict__ decay, int H,
                                                float* __restrict__ cv, float* __restrict__ ab) {
    const int row = blockIdx.x, c0 = blockIdx.y * chunk, c1 = min(ch, c0 + chunk);
    const float* pr = proj + (size_t)row * ldp + off;
    if (((ldp | off | ch | chunk) & 3) == 0) {          // 16-byte rows: four channels per thread
        for (int c = c0 + threadIdx.x * 4; c < c1; c += blockDim.x * 4) {
            float t[4];
            ld_vec<4>(pr + c, t);
#pragma unroll
            for (int i = 0; i < 4; ++i) t[i] = siluf_(t[i]);
            st_vec<4>(cv + (size_t)row * ch + c, t);
        }
    } else {
        for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) cv[(size_t)row * ch + c] = siluf_(pr[c]);
    }
    if (blockIdx.y != 0) return;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        ab[((size_t)row * H + h) * 2] = decay[h];
        ab[((size_t)row * H + h) * 2 + 1] = 1.f;
    }
}

// The input convolution in front of a sublayer: out[row, c] = in[row, c] + sum_k w[c, k] * in[position - (taps - 1 - k), c] (no bias,
// no activation; a.proj / a.off name `in`), with its hi | lo halves.  grid (row blocks of `rpb` rows, channel blocks); a thread takes V
// consecutive channels (V = 4: 16-byte accesses; ch, ldp and off multiples of 4) through the block's rows in turn and keeps its
// channels' taps in its own shared-memory cells ([taps][threads][V] floats: no barrier is needed).
template <int V>
static __global__ void __launch_bounds__(128) ly_input_conv_kernel(ConvArgs a, int rpb, int T, float* __restrict__ out, uint16_t* __restrict__ ohi,
                                                                     uint16_t* __restrict__ olo) {
    extern __shared__ __align__(16) float wsm[];
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= a.ch) return;
    for (int k = 0; k < a.taps; ++k)
#pragma unroll
        for (int i = 0; i < V; ++i) wsm[((size_t)k * blockDim.x + threadIdx.x) * V + i] = a.w[(size_t)(c + i) * a.taps + k];
    const int r_hi = min(T, (int)(blockIdx.x + 1) * rpb);
    for (int row = blockIdx.x * rpb; row < r_hi; ++row) {
        const int seq = a.row_seq[row], pos = a.row_pos[row];
        const int row0 = a.seq_row0[seq], pos0 = a.seq_pos0[seq], slot = a.seq_slot[seq];
        float t[V];
#pragma unroll
        for (int i = 0; i < V; ++i) t[i] = 0.f;
        for (int k = 0; k < a.taps; ++k) {
            const int back = a.taps - 1 - k;
            const float* src;
            if (row - back >= row0) src = a.proj + (size_t)(row - back) * a.ldp + a.off;
            else {
                const int p = pos - back;
                if (p < 0) continue;                 // before the sequence's start: zeros
                src = a.state + ((size_t)slot * (a.taps - 1) + (p - pos0 + a.taps - 1)) * a.ch;
            }
            float in[V], wk[V];
            ld_vec<V>(src + c, in); ld_vec<V>(wsm + ((size_t)k * blockDim.x + threadIdx.x) * V, wk);
#pragma unroll
            for (int i = 0; i < V; ++i) t[i] = fmaf(wk[i], in[i], t[i]);
        }
        float self[V];
        ld_vec<V>(a.proj + (size_t)row * a.ldp + a.off + c, self);
#pragma unroll
        for (int i = 0; i < V; ++i) t[i] += self[i];
        st_vec<V>(out + (size_t)row * a.ch + c, t);
        split_store_vec<V>(ohi, olo, (size_t)row * a.ch + c, t);
    }
}

// Mamba-2, per row: x | B | C <- silu(conv + bias);  per head  b = softplus(dt + dt_bias),  a = exp(-exp(A_log) b)  -> ab[row, h] = (a, b).
// grid (rows, channel chunks of `chunk`): the first chunk's block also computes the per-head scalars.
static __global__ void ly_mamba_prep_kernel(ConvArgs a, int chunk, int off_dt, const float* __restrict__ dt_bias, const float* __restrict__ a_log, int H,
                                            float* __restrict__ ab) {
    const int row = blockIdx.x, seq = a.row_seq[row], pos = a.row_pos[row];
    const int row0 = a.seq_row0[seq], pos0 = a.seq_pos0[seq], slot = a.seq_slot[seq];
    const int c0 = blockIdx.y * chunk, c1 = min(a.ch, c0 + chunk);
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) a.cv[(size_t)row * a.ch + c] = conv_silu(a, row, row0, pos, pos0, slot, c);
    if (blockIdx.y != 0) return;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float dt = softplusf_(a.proj[(size_t)row * a.ldp + off_dt + h] + dt_bias[h]);
        ab[((size_t)row * H + h) * 2] = expf(-expf(a_log[h]) * dt);
        ab[((size_t)row * H + h) * 2 + 1] = dt;
    }
}

// Gated delta rule, per row: q | k | v <- silu(conv);  q, k heads -> unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times qscale;
// per head  b = sigmoid(proj[off_b + h]),  a = exp(-exp(A_log) softplus(proj[off_a + h] + dt_bias))  -> ab[row, h] = (a, b).
// grid (rows, channel chunks of `chunk`, a multiple of D: a q or k head never straddles two blocks).
static __global__ void ly_delta_prep_kernel(ConvArgs a, int chunk, int off_b, int off_a, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                            int H, int G, int D, float qscale, float* __restrict__ ab) {
    const int row = blockIdx.x, seq = a.row_seq[row], pos = a.row_pos[row];
    const int row0 = a.seq_row0[seq], pos0 = a.seq_pos0[seq], slot = a.seq_slot[seq];
    const int c0 = blockIdx.y * chunk, c1 = min(a.ch, c0 + chunk);
    float* cvr = a.cv + (size_t)row * a.ch;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) cvr[c] = conv_silu(a, row, row0, pos, pos0, slot, c);
    if (blockIdx.y == 0) {
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const float* pr = a.proj + (size_t)row * a.ldp;
            ab[((size_t)row * H + h) * 2] = expf(-expf(a_log[h]) * softplusf_(pr[off_a + h] + dt_bias[h]));
            ab[((size_t)row * H + h) * 2 + 1] = sigmoidf_(pr[off_b + h]);
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int h0 = c0 / D, h1 = min(2 * G, c1 / D);         // q heads, then k heads, of this chunk
    for (int it = h0 + wid; it < h1; it += nw) {
        float* v = cvr + (size_t)it * D;
        float ss = 0.f;
        for (int c = lane; c < D; c += 32) ss += v[c] * v[c];
        const float r = (it < G ? qscale : 1.f) / sqrtf(warp_sum(ss) + 1e-6f);
        for (int c = lane; c < D; c += 32) v[c] *= r;
    }
}

struct RecArgs {
    const float* cv; int ldc, off_q, off_k, off_v;      // read-out vector q[g], write vector k[g] (D channels each), value v[h] (Dv channels)
    const float* ab;            // [T, H, 2]: decay a, strength b
    const float* dskip;         // [H] or nullptr: o += dskip[h] * v
    float* o;                   // [T, H * Dv]
    float* state;               // [slots][H][D][Dv]
    const int *seq_row0, *seq_slot, *seq_pos0;
    int H, G, D, Dv;
};
constexpr int kRecCols = 32, kRecParts = 4;       // value columns per block; threads that share a column's rows
// Token by token, per head:  S <- a S;  u = b v   (DELTA: u = b (v - S^T k));  S <- S + k u^T;  o = S^T q (+ dskip v).
// One block of four warps per (sequence, head, 32 value columns) -- columns of S never interact.  A column's rows are split over
// four neighbouring lanes (lane part p keeps rows p RPT .. p RPT + RPT - 1 in registers), so the two reductions over rows are a
// serial sum per lane and two shuffles: the warps of a block never wait for one another.  Each warp keeps a ring of the next
// tokens' operands (k, q, its eight values, a, b) in its own shared memory, filled by asynchronous copies several tokens ahead,
// so a token's step waits for no global load.  The order of operations per token does not depend on how a prompt was cut.
template <int RPT, bool DELTA>
static __global__ void __launch_bounds__(128) ly_rec_scan_kernel(RecArgs a) {
    extern __shared__ __align__(16) float sm[]; // [4 warps][NST tokens][k | q: 4 parts x (RPT + 4) each (the pad keeps the parts on different banks) | v x 8 | a | b | pad]
    constexpr int DP = RPT * kRecParts;         // rows, padded (rows >= D hold zeros and never change)
    constexpr int PS = RPT + 4, DPS = kRecParts * PS;      // floats per part / per vector in shared memory
    constexpr int NST = RPT >= 64 ? 4 : 8;      // tokens in the ring
    constexpr int SLOT = 2 * DPS + 12;
    constexpr int NL = (2 * DP + 31) / 32;      // k | q values a lane copies per token
    const int D = a.D, Dv = a.Dv;
    const int seq = blockIdx.x, hd = blockIdx.y, g = hd / (a.H / a.G);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, p = lane & 3, cl = lane >> 2;
    const int col0 = blockIdx.z * kRecCols + wid * 8, col = col0 + cl;
    const bool vok = col < Dv;
    float* wsm = sm + wid * (NST * SLOT);
    const int r0 = a.seq_row0[seq], r1 = a.seq_row0[seq + 1];
    float* st = a.state + (((size_t)a.seq_slot[seq] * a.H + hd) * D) * Dv + col;
    float s[RPT];
    const bool fresh = a.seq_pos0[seq] == 0;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int d = p * RPT + i;
        s[i] = (!fresh && vok && d < D) ? st[(size_t)d * Dv] : 0.f;
    }
    const float dsk = a.dskip ? a.dskip[hd] : 0.f;
    for (int i = lane; i < NST * SLOT; i += 32) wsm[i] = 0.f;       // what no copy ever writes (rows >= D, columns >= Dv) reads as zero
    __syncwarp();
    auto issue = [&](int row, int slot) {
        const float* pr = a.cv + (size_t)row * a.ldc;
        float* dst = wsm + slot * SLOT;
#pragma unroll
        for (int t = 0; t < NL; ++t) {
            const int idx = lane + 32 * t, isq = idx >= DP, d = idx - isq * DP;
            if (idx < 2 * DP && d < D) cp_async_f32(dst + isq * DPS + (d / RPT) * PS + d % RPT, pr + (isq ? a.off_q : a.off_k) + g * D + d);
        }
        if (lane < 8) {
            if (col0 + lane < Dv) cp_async_f32(dst + 2 * DPS + lane, pr + a.off_v + hd * Dv + col0 + lane);
        } else if (lane < 10) {
            cp_async_f32(dst + 2 * DPS + lane, a.ab + ((size_t)row * a.H + hd) * 2 + (lane - 8));
        }
    };
#pragma unroll
    for (int t = 0; t < NST - 1; ++t) {
        if (r0 + t < r1) issue(r0 + t, t);
        cp_async_commit();
    }
    int it = 0;
    for (int row = r0; row < r1; ++row, ++it) {
        if (row + NST - 1 < r1) issue(row + NST - 1, (it + NST - 1) % NST);
        cp_async_commit();
        cp_async_wait<NST - 1>();               // this token's copies have landed (one group per token, empty ones included)
        __syncwarp();
        const float* cur = wsm + (it % NST) * SLOT;
        const float v = cur[2 * DPS + cl], da = cur[2 * DPS + 8], db = cur[2 * DPS + 9];
        float kb[RPT], qb[RPT];                 // this lane's rows of k and q
        {
            const float* ks = cur + p * PS;
            if (RPT % 4 == 0) {
#pragma unroll
                for (int i = 0; i < RPT / 4; ++i) {
                    const float4 k4 = reinterpret_cast<const float4*>(ks)[i], q4 = reinterpret_cast<const float4*>(ks + DPS)[i];
                    kb[4 * i] = k4.x; kb[4 * i + 1] = k4.y; kb[4 * i + 2] = k4.z; kb[4 * i + 3] = k4.w;
                    qb[4 * i] = q4.x; qb[4 * i + 1] = q4.y; qb[4 * i + 2] = q4.z; qb[4 * i + 3] = q4.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < RPT; ++i) { kb[i] = ks[i]; qb[i] = ks[DPS + i]; }
            }
        }
        float u;
        if (DELTA) {
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; ++i) { s[i] *= da; part = fmaf(s[i], kb[i], part); }
            part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
            part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
            u = db * (v - part);
        } else {
#pragma unroll
            for (int i = 0; i < RPT; ++i) s[i] *= da;
            u = db * v;
        }
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            s[i] = fmaf(kb[i], u, s[i]);
            acc = fmaf(s[i], qb[i], acc);
        }
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
        if (p == 0 && vok) a.o[(size_t)row * a.H * Dv + hd * Dv + col] = acc + dsk * v;
        __syncwarp();                           // the slot may be refilled in the next iteration
    }
    cp_async_wait<0>();
    if (vok) {
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int d = p * RPT + i;
            if (d < D) st[(size_t)d * Dv] = s[i];
        }
    }
}

// u[row, part] = v / sqrt(mean_part v^2 + eps) * w,  v = y * silu(z): the gated output of Mamba-2, normed in `parts` equal pieces of
// the inner width.  z = proj[row, off_z ...].  One block per (row, part).
// sig_after: u[row, part] = y / sqrt(mean_part y^2 + eps) * w * sigmoid(z) instead -- the norm sees the scan's output itself and the
// gate follows it (lightning attention, parts = 1).
static __global__ void ly_gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ proj, int ldp, int off_z,
                                                  const float* __restrict__ w, float eps, int inner, int parts, int sig_after, float* __restrict__ u,
                                                  uint16_t* __restrict__ uhi, uint16_t* __restrict__ ulo) {
    __shared__ float red[33];
    const int row = blockIdx.x, n = inner / parts, c0 = blockIdx.y * n;
    const float* yr = y + (size_t)row * inner + c0;
    const float* zr = proj + (size_t)row * ldp + off_z + c0;
    if (((inner | n | ldp | off_z) & 3) == 0) {         // 16-byte rows and parts: four channels per thread
        float ss = 0.f;
        for (int c = threadIdx.x * 4; c < n; c += blockDim.x * 4) {
            float a[4], z[4];
            ld_vec<4>(yr + c, a);
            if (!sig_after) {
                ld_vec<4>(zr + c, z);
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] *= siluf_(z[i]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) ss += a[i] * a[i];
        }
        const float r = 1.f / sqrtf(block_sum(ss, red) / (float)n + eps);
        for (int c = threadIdx.x * 4; c < n; c += blockDim.x * 4) {
            float a[4], z[4], ww[4];
            ld_vec<4>(yr + c, a); ld_vec<4>(zr + c, z); ld_vec<4>(w + c0 + c, ww);
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sig_after ? a[i] * r * ww[i] * sigmoidf_(z[i]) : a[i] * siluf_(z[i]) * r * ww[i];
            st_vec<4>(u + (size_t)row * inner + c0 + c, a);
            split_store_vec<4>(uhi, ulo, (size_t)row * inner + c0 + c, a);
        }
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = sig_after ? yr[c] : yr[c] * siluf_(zr[c]); ss += v * v; }
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = sig_after ? yr[c] * r * w[c0 + c] * sigmoidf_(zr[c]) : yr[c] * siluf_(zr[c]) * r * w[c0 + c];
        u[(size_t)row * inner + c0 + c] = v;
        split_store(uhi, ulo, (size_t)row * inner + c0 + c, v);
    }
}

// ---- feed-forward ----------------------------------------------------------------------------------------------------------
// act 0: act[p, f] = g * sigmoid(1.702 g) * (u + 1),  g = min(gu[p, f], limit),  u = clamp(gu[p, F + f], -limit, limit);
// act 1: act[p, f] = gelu_tanh(g) * u,  gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  bias [2F] (optional) is added
// to gate | up first.  act 2: act[p, f] = relu(gu[p, f])^2 -- no gate matrix, gu has F columns.  act 3: act[p, f] = relu(g) * u.  p < *count
__device__ __forceinline__ float glu_value(float g, float u, int act, float limit) {
    if (act == 2) { g = fmaxf(g, 0.f); return g * g; }
    if (act == 3) return fmaxf(g, 0.f) * u;
    if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoidf_(1.702f * g) * (u + 1.f);
}
static __global__ void ly_glu_kernel(const float* __restrict__ gu, int F, float limit, int act_kind, const float* __restrict__ bias,
                                     const int* __restrict__ count, int rows, float* __restrict__ act, uint16_t* __restrict__ ahi,
                                     uint16_t* __restrict__ alo) {
    const int n = count ? *count : rows;
    const size_t total = (size_t)n * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t p = i / F, f = i - p * F;
        const size_t gs = act_kind == 2 ? (size_t)F : (size_t)2 * F;
        const float g = gu[p * gs + f] + (bias ? bias[f] : 0.f);
        const float u = act_kind == 2 ? 0.f : gu[p * gs + F + f] + (bias ? bias[F + f] : 0.f);
        const float v = glu_value(g, u, act_kind, limit);
        if (act != nullptr) act[i] = v;         // nullptr: only the hi | lo halves are consumed (a tensor-core GEMM follows)
        split_store(ahi, alo, i, v);
    }
}

// Router: z = Wr h (f32), s = softmax(z) over all experts, the `top` largest (lower index first among equals), weights s / (sum + 1e-20).
// Also the shared expert's gate sigmoid(w_sg . h).  One block per row, one warp per expert in turn.
// rb (optional): a bias [E] added to the logits.  (Softmax over all, then renormalised over the chosen = softmax over the chosen alone.)
static __global__ void ly_router_kernel(const float* __restrict__ h, int W, const float* __restrict__ wr, const float* __restrict__ rb, int E, int top,
                                        const float* __restrict__ wsg, int* __restrict__ sel, float* __restrict__ wt, float* __restrict__ sgate) {
    extern __shared__ float z[];                 // [E]
    const int row = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* hr = h + (size_t)row * W;
    for (int e = wid; e <= E; e += nw) {
        if (e == E && wsg == nullptr) break;
        const float* w = e < E ? wr + (size_t)e * W : wsg;
        float d = 0.f;
        if ((W & 3) == 0) {         // 16-byte rows: four channels per load
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* h4 = reinterpret_cast<const float4*>(hr);
            for (int c = lane; c < W / 4; c += 32) {
                const float4 a = w4[c], b = h4[c];
                d = fmaf(a.x, b.x, d); d = fmaf(a.y, b.y, d); d = fmaf(a.z, b.z, d); d = fmaf(a.w, b.w, d);
            }
        } else {
            for (int c = lane; c < W; c += 32) d = fmaf(w[c], hr[c], d);
        }
        d = warp_sum(d);
        if (lane == 0) {
            if (e < E) z[e] = d + (rb ? rb[e] : 0.f); else sgate[row] = sigmoidf_(d);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float mx = -INFINITY;
        for (int e = 0; e < E; ++e) mx = fmaxf(mx, z[e]);
        float sum = 0.f;
        for (int e = 0; e < E; ++e) { z[e] = expf(z[e] - mx); sum += z[e]; }
        const float inv = 1.f / sum;
        float psum = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float bv = -1.f;
            for (int e = 0; e < E; ++e)
                if (z[e] > bv) { bv = z[e]; best = e; }
            sel[row * top + k] = best;
            wt[row * top + k] = bv * inv;
            psum += bv * inv;
            z[best] = -2.f;
        }
        const float pinv = 1.f / (psum + 1e-20f);
        for (int k = 0; k < top; ++k) wt[row * top + k] *= pinv;
    }
}

// Router with independent scores: z = Wr h (f32), s = sigmoid(z); the choice runs on c = s + corr.  The experts form `groups` equal
// groups of neighbours; a group's mark is the sum of its two largest c (its only one, for groups of one); the `keep` groups with the
// largest marks stay eligible, the others' experts cannot be chosen whatever their c (c may be negative); the `top` eligible experts
// with the largest c are used with the weights s, as they are.  Lower index first among equals, everywhere.
// One block per row, one warp per expert in turn; shared memory: 2 E + groups floats.
static __global__ void ly_router_sigmoid_kernel(const float* __restrict__ h, int W, const float* __restrict__ wr, int E, int top,
                                                const float* __restrict__ corr, int groups, int keep, int* __restrict__ sel,
                                                float* __restrict__ wt) {
    extern __shared__ float z[];                 // [E] scores s, [E] choice scores c, [groups] marks
    float* cc = z + E;
    float* mark = cc + E;
    const int row = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* hr = h + (size_t)row * W;
    for (int e = wid; e < E; e += nw) {
        const float* w = wr + (size_t)e * W;
        float d = 0.f;
        if ((W & 3) == 0) {
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* h4 = reinterpret_cast<const float4*>(hr);
            for (int c = lane; c < W / 4; c += 32) {
                const float4 a = w4[c], b = h4[c];
                d = fmaf(a.x, b.x, d); d = fmaf(a.y, b.y, d); d = fmaf(a.z, b.z, d); d = fmaf(a.w, b.w, d);
            }
        } else {
            for (int c = lane; c < W; c += 32) d = fmaf(w[c], hr[c], d);
        }
        d = warp_sum(d);
        if (lane == 0) { const float s = sigmoidf_(d); z[e] = s; cc[e] = s + corr[e]; }
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    const int per = E / groups;
    for (int g = 0; g < groups; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) {
            const float v = cc[e];
            if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v;
        }
        mark[g] = per > 1 ? b1 + b2 : b1;
    }
    // drop the groups.count - keep groups with the smallest marks (higher index first among equals): what stays is the `keep` best
    for (int k = 0; k < groups - keep; ++k) {
        int worst = -1;
        float wv = INFINITY;
        for (int g = 0; g < groups; ++g)
            if (mark[g] != INFINITY && (worst < 0 || mark[g] <= wv)) { wv = mark[g]; worst = g; }
        mark[worst] = INFINITY;                  // a dropped group
        for (int e = worst * per; e < (worst + 1) * per; ++e) cc[e] = -INFINITY;
    }
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float bv = -INFINITY;
        for (int e = 0; e < E; ++e)
            if (cc[e] > bv) { bv = cc[e]; best = e; }
        if (best < 0) best = 0;                  // only with scores that are not numbers
        sel[row * top + k] = best;
        wt[row * top + k] = z[best];
        cc[best] = -INFINITY;
    }
}

// Row lists per expert, in ascending (row, pick) order: grp_off[E + 1], pair_row[p] = source row, pair_of[row * top + k] = p.
// One warp per expert (grid = E blocks of 32 threads): a first sweep counts the picks of lower experts (the list's offset) and
// its own, a second places its picks by ballot compaction -- stable, so the lists do not depend on timing.
static __global__ void ly_moe_lists_kernel(const int* __restrict__ sel, int T, int top, int E, int* __restrict__ grp_off, int* __restrict__ pair_row,
                                           int* __restrict__ pair_of) {
    const int e = blockIdx.x, lane = threadIdx.x, n = T * top;
    int less = 0, mine = 0;
    for (int i = lane; i < n; i += 32) {
        const int s = sel[i];
        less += s < e;
        mine += s == e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { less += __shfl_xor_sync(0xFFFFFFFFu, less, o); mine += __shfl_xor_sync(0xFFFFFFFFu, mine, o); }
    if (lane == 0) {
        grp_off[e] = less;
        if (e == E - 1) grp_off[E] = less + mine;
    }
    int p = less;
    for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        const bool hit = i < n && sel[i] == e;
        const unsigned m = __ballot_sync(0xFFFFFFFFu, hit);
        if (hit) {
            const int q = p + __popc(m & ((1u << lane) - 1u));
            pair_row[q] = i / top;
            pair_of[i] = q;
        }
        p += __popc(m);
    }
}

// ---- experts on the tensor-core GEMMs (serving precision) --------------------------------------------------------------------
// Few rows (every expert's list fits one block of `cap` rows): block e of gx_hi / gx_lo = the hi | lo halves of the rows routed to
// expert e, in list order; cnt[e] = their number.  grid (E, row workers).
static __global__ void ly_moe_gather_kernel(const uint16_t* __restrict__ hhi, const uint16_t* __restrict__ hlo, int W, const int* __restrict__ grp_off,
                                            const int* __restrict__ pair_row, int cap, uint16_t* __restrict__ gx_hi, uint16_t* __restrict__ gx_lo,
                                            int* __restrict__ cnt) {
    const int e = blockIdx.x, lo = grp_off[e], n = grp_off[e + 1] - lo;
    if (blockIdx.y == 0 && threadIdx.x == 0) cnt[e] = n;
    for (int i = blockIdx.y; i < n; i += gridDim.y) {
        const size_t src = (size_t)pair_row[lo + i] * W, dst = ((size_t)e * cap + i) * W;
        for (int c = threadIdx.x; c < W; c += blockDim.x) { gx_hi[dst + c] = hhi[src + c]; gx_lo[dst + c] = hlo[src + c]; }
    }
}
// The activation over the grouped GEMM's output: gu[slice][e * cap + i][2F] (F columns for the ungated act 2) summed over slices, rows
// i < cnt[e] only -> hi | lo.
static __global__ void ly_glu_grouped_kernel(const float* __restrict__ gu, int nsl, size_t sl_stride, int F, float limit, int act_kind,
                                             const int* __restrict__ cnt, int cap, uint16_t* __restrict__ ahi, uint16_t* __restrict__ alo) {
    const int r = blockIdx.y;                   // row e * cap + i
    if (r % cap >= cnt[r / cap]) return;
    for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < F; f += gridDim.x * blockDim.x) {
        float g = 0.f, u = 0.f;
        const size_t gs = act_kind == 2 ? (size_t)F : (size_t)2 * F;
        for (int k = 0; k < nsl; ++k) {
            g += gu[k * sl_stride + (size_t)r * gs + f];
            if (act_kind != 2) u += gu[k * sl_stride + (size_t)r * gs + F + f];
        }
        split_store(ahi, alo, (size_t)r * F + f, glu_value(g, u, act_kind, limit));
    }
}
// y[row, c] = sum_k wt[row, k] * (sum over slices of eo[slice][block row of (row, k)][c]) + sgate[row] * sh[row, c]
static __global__ void ly_moe_combine_grouped_kernel(const float* __restrict__ eo, int nsl, size_t sl_stride, const int* __restrict__ sel,
                                                     const int* __restrict__ pair_of, const int* __restrict__ grp_off, int cap,
                                                     const float* __restrict__ wt, int top, const float* __restrict__ sh, const float* __restrict__ sgate,
                                                     int W, float* __restrict__ y) {
    const int row = blockIdx.y;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < W; c += gridDim.x * blockDim.x) {
        float t = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = sel[row * top + k];
            const size_t r = (size_t)e * cap + (pair_of[row * top + k] - grp_off[e]);
            float v = 0.f;
            for (int sl = 0; sl < nsl; ++sl) v += eo[sl * sl_stride + r * W + c];
            t = fmaf(wt[row * top + k], v, t);
        }
        if (sh != nullptr) t = fmaf(sgate ? sgate[row] : 1.f, sh[(size_t)row * W + c], t);
        y[(size_t)row * W + c] = t;
    }
}
// Many rows: every expert runs over ALL rows on the tensor cores and a row keeps expert e's output times its routing weight (zero
// when it did not pick e).  y (+)= w_e[row] * ye[row];  e < 0: the shared expert, weight sgate[row].  Experts in ascending order.
static __global__ void ly_moe_accum_kernel(const float* __restrict__ ye, const int* __restrict__ sel, const float* __restrict__ wt, int top, int e,
                                           const float* __restrict__ sgate, int first, int W, float* __restrict__ y) {
    const int row = blockIdx.y;
    float w = 0.f;
    if (e < 0) w = sgate ? sgate[row] : 1.f;
    else
        for (int k = 0; k < top; ++k) w += sel[row * top + k] == e ? wt[row * top + k] : 0.f;
    if (w == 0.f && !first) return;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < W; c += gridDim.x * blockDim.x) {
        const size_t i = (size_t)row * W + c;
        const float add = w != 0.f ? w * ye[i] : 0.f;
        y[i] = first ? add : y[i] + add;
    }
}

// y[row, c] = sum_k wt[row, k] * eo[pair_of[row, k], c]  (pick order)  + sgate[row] * sh[row, c]
static __global__ void ly_moe_combine_kernel(const float* __restrict__ eo, const int* __restrict__ pair_of, const float* __restrict__ wt, int top,
                                             const float* __restrict__ sh, const float* __restrict__ sgate, int W, float* __restrict__ y) {
    const int row = blockIdx.y;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < W; c += gridDim.x * blockDim.x) {
        float t = 0.f;
        for (int k = 0; k < top; ++k) t = fmaf(wt[row * top + k], eo[(size_t)pair_of[row * top + k] * W + c], t);
        if (sh != nullptr) t = fmaf(sgate ? sgate[row] : 1.f, sh[(size_t)row * W + c], t);
        y[(size_t)row * W + c] = t;
    }
}

}  // namespace fl
