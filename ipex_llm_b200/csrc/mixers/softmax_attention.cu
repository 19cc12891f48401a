// Causal softmax attention over keys and values that are addressed by strides, and the preparation of a latent cache.
//   latent_prepare: RMS norm (plain weight) of two column ranges of one projection output: the query latent goes to a dense
//     buffer, the key/value latent is appended to the cache (one vector per position, shared by all heads);
//   softmax_attention: scores, softmax and the weighted sum of values with 32-bit scores and weights.  Keys and values are
//     [batch, position, kv head, channel] tensors given by three strides each, so the same kernels serve keys / values
//     expanded from the latent (one row per head) and the latent cache itself read as one shared key = value head of
//     kv_rank channels (the "absorbed" form: the query carries the key expansion, the value expansion follows the sum).
//   An optional window limits how far back a query looks (0 = every earlier position), optional chunks confine a query to the
//   earlier positions of its own chunk (chunks counted from the row's first token); scores may be soft-capped
//   (cap * tanh(score / cap)) and the softmax's denominator may hold a per-head sink exp(sink_h) that has no key and no value.
//   wide_qkv_prepare: RMS norm over a token's WHOLE query projection and whole key projection (all heads at once, one weight per
//     channel), values optionally blended with another layer's values of the same token; keys and values are appended to the
//     cache.
#include "mixers_common.cuh"
#include <math.h>

// one block of 128 threads per (token, segment): segment 0 = query latent, 1 = key/value latent.  Segments up to 1024 wide are
// held in registers (one round of loads); wider ones are read twice.
constexpr int LP_THREADS = 128, LP_MAXC = 8;
template <typename T>
__global__ void __launch_bounds__(LP_THREADS) latent_prepare_kernel(
        const T* __restrict__ proj, int B, int S, int ld, int off_q, int q_rank, const T* __restrict__ q_w, int off_c, int kv_rank,
        const T* __restrict__ c_w, float eps, T* __restrict__ cq_out, T* __restrict__ store, int cap, int held, int shift,
        const int32_t* __restrict__ pad, const int32_t* __restrict__ dyn) {
    __shared__ float red[LP_THREADS / 32];
    if (dyn) held = dyn[0];
    const long n = blockIdx.x >> 1;
    const int seg = blockIdx.x & 1;
    const int b = (int)(n / S), t = (int)(n - (long)b * S);
    const bool real = held + t + shift - pad[b] >= 0;       // padding slots hold zeros
    const int width = seg ? kv_rank : q_rank;
    if (width == 0) return;
    const T* src = proj + n * (long)ld + (seg ? off_c : off_q);
    const T* w = seg ? c_w : q_w;
    T* dst = seg ? store + ((long)b * cap + held + t) * kv_rank : cq_out + n * (long)q_rank;
    const bool cached = width <= LP_MAXC * LP_THREADS;
    float sv[LP_MAXC], wv[LP_MAXC];
    float ss = 0.0f;
    if (cached) {
#pragma unroll
        for (int k = 0; k < LP_MAXC; ++k) {
            const int c = threadIdx.x + k * LP_THREADS;
            sv[k] = c < width ? to_f(src[c]) : 0.0f;
            wv[k] = c < width ? to_f(w[c]) : 0.0f;
            ss += sv[k] * sv[k];
        }
    } else {
        for (int c = threadIdx.x; c < width; c += LP_THREADS) { float v = to_f(src[c]); ss += v * v; }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.0f;
#pragma unroll
    for (int i = 0; i < LP_THREADS / 32; ++i) ss += red[i];
    const float inv = real ? 1.0f / sqrtf(ss / (float)width + eps) : 0.0f;
    if (cached) {
#pragma unroll
        for (int k = 0; k < LP_MAXC; ++k) {
            const int c = threadIdx.x + k * LP_THREADS;
            if (c < width) dst[c] = from_f<T>(sv[k] * inv * wv[k]);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += LP_THREADS) dst[c] = from_f<T>(to_f(src[c]) * inv * to_f(w[c]));
    }
}

// one block per (token, segment): 0 = queries (norm over heads * dim channels -> q_out), 1 = keys (norm over kv_heads * dim
// channels -> cache), 2 = values ((1 - blend) v + blend v_other when v_other is given -> cache).  Padding slots store zeros.
// a segment that fits QP_MAXC elements a thread is held in registers; a prompt's many tokens run in blocks of 128 threads, the few
// tokens of a decoding step in blocks of up to 1024 so that projections up to 8192 wide take one round trip to memory
constexpr int QP_MAXC = 8, QP_FEW_TOKENS = 64;
template <typename T, int QP_THREADS>
__global__ void __launch_bounds__(QP_THREADS) wide_qkv_prepare_kernel(
        const T* __restrict__ proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads, int dim, int vdim,
        const T* __restrict__ q_w, const T* __restrict__ k_w, float eps, const T* __restrict__ v_other, long ld_other, const T* __restrict__ blend,
        T* __restrict__ q_out, T* __restrict__ k_store, T* __restrict__ v_store, int cap, int held, int shift, const int32_t* __restrict__ pad,
        const int32_t* __restrict__ dyn) {
    __shared__ float red[QP_THREADS / 32];
    if (dyn) held = dyn[0];
    const long n = blockIdx.x / 3;
    const int seg = blockIdx.x - 3 * n;
    const int b = (int)(n / S), t = (int)(n - (long)b * S);
    const bool real = held + t + shift - pad[b] >= 0;
    const T* row = proj + n * (long)ld;
    if (seg == 2) {
        const int width = kv_heads * vdim;
        const float lam = v_other ? to_f(blend[0]) : 0.0f;
        for (int c = threadIdx.x; c < width; c += QP_THREADS) {
            float v = to_f(row[off_v + c]);
            if (v_other) v = (1.0f - lam) * v + lam * to_f(v_other[n * ld_other + c]);
            const int g = c / vdim;
            v_store[(((long)b * kv_heads + g) * cap + held + t) * vdim + (c - g * vdim)] = from_f<T>(real ? v : 0.0f);
        }
        return;
    }
    const int hd = seg ? kv_heads : heads;
    const int width = hd * dim;
    const T* src = row + (seg ? off_k : off_q);
    const T* w = seg ? k_w : q_w;
    const bool cached = width <= QP_MAXC * QP_THREADS;
    float sv[QP_MAXC];
    float ss = 0.0f;
    if (cached) {
#pragma unroll
        for (int k = 0; k < QP_MAXC; ++k) {
            const int c = threadIdx.x + k * QP_THREADS;
            sv[k] = c < width ? to_f(src[c]) : 0.0f;
            ss += sv[k] * sv[k];
        }
    } else {
        for (int c = threadIdx.x; c < width; c += QP_THREADS) { float v = to_f(src[c]); ss += v * v; }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.0f;
#pragma unroll
    for (int i = 0; i < QP_THREADS / 32; ++i) ss += red[i];
    const float inv = real ? 1.0f / sqrtf(ss / (float)width + eps) : 0.0f;
    auto put = [&](int c, float v) {
        const float y = v * inv * to_f(w[c]);
        if (seg == 0) { q_out[n * (long)width + c] = from_f<T>(y); return; }
        const int g = c / dim;
        k_store[(((long)b * kv_heads + g) * cap + held + t) * dim + (c - g * dim)] = from_f<T>(y);
    };
    if (cached) {
#pragma unroll
        for (int k = 0; k < QP_MAXC; ++k) {
            const int c = threadIdx.x + k * QP_THREADS;
            if (c < width) put(c, sv[k]);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += QP_THREADS) put(c, to_f(src[c]));
    }
}

// Rotary positions on the queries and keys of new tokens, taken from the columns of one projection output, with the cache write
// of keys and values: one warp per (token, head slot) -- `heads` query heads of q_dim channels, `kv_heads` key heads of k_dim
// channels and, when vdim > 0, `kv_heads` value heads.  Inside a head, channel rot_off + i is paired with channel
// rot_off + i + rot_dims / 2 (i < rot_dims / 2) and the pair (u, v) becomes (u cos a - v sin a, v cos a + u sin a) * amp with
// a = position * inv_freq[i], the angle and its sine / cosine in double precision; the other channels pass unchanged.  The first
// k_norm_cols channels of a key head are first divided by their root mean square and multiplied by k_norm_w (a latent that
// shares its cache row with a rotated part).  Keys and values go to storage index held + t of caches given by three strides.
template <typename T>
__global__ void rope_qk_prepare_kernel(const T* __restrict__ proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads,
                                       int q_dim, int k_dim, int vdim, int q_rot_off, int k_rot_off, int rot_dims, const double* __restrict__ inv_freq,
                                       float amp, const T* __restrict__ k_norm_w, int k_norm_cols, float eps, T* __restrict__ q_out,
                                       T* __restrict__ k_store, long k_bs, long k_ps, long k_hs, T* __restrict__ v_store, long v_bs, long v_ps,
                                       long v_hs, int held, int shift, const int32_t* __restrict__ pad, const int32_t* __restrict__ dyn) {
    if (dyn) held = dyn[0];
    const int slots = heads + kv_heads + (vdim > 0 ? kv_heads : 0);
    const long warp = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long)B * S * slots) return;
    const long n = warp / slots;
    const int hs = (int)(warp - n * slots);
    const int b = (int)(n / S), t = (int)(n - (long)b * S);
    const int pos = held + t + shift - pad[b];              // negative: a padding slot
    const T* row = proj + n * (long)ld;
    if (hs >= heads + kv_heads) {
        const int g = hs - heads - kv_heads;
        const T* src = row + off_v + g * vdim;
        T* dst = v_store + b * v_bs + (long)(held + t) * v_ps + g * v_hs;
        for (int c = lane; c < vdim; c += 32) dst[c] = pos >= 0 ? src[c] : from_f<T>(0.0f);
        return;
    }
    const bool is_q = hs < heads;
    const int g = is_q ? hs : hs - heads;
    const int dim = is_q ? q_dim : k_dim, rot_off = is_q ? q_rot_off : k_rot_off;
    const T* src = row + (is_q ? off_q : off_k) + g * dim;
    T* dst = is_q ? q_out + (n * heads + g) * (long)dim : k_store + b * k_bs + (long)(held + t) * k_ps + g * k_hs;
    const int ncols = (!is_q && k_norm_w) ? k_norm_cols : 0;
    float inv = 1.0f;
    if (ncols > 0) {
        float ss = 0.0f;
        for (int c = lane; c < ncols; c += 32) { const float v = to_f(src[c]); ss += v * v; }
        inv = 1.0f / sqrtf(warp_sum(ss) / (float)ncols + eps);
    }
    const int half = rot_dims >> 1;
    const double dpos = (double)pos;
    for (int c = lane; c < dim; c += 32) {
        const int r = c - rot_off;
        float y;
        if (r >= 0 && r < rot_dims) {
            const int i = r < half ? r : r - half;
            double dsn, dcs;
            sincos(dpos * inv_freq[i], &dsn, &dcs);
            const float sn = (float)dsn * amp, cs = (float)dcs * amp;
            const float u = to_f(src[rot_off + i]), v = to_f(src[rot_off + i + half]);
            y = r < half ? u * cs - v * sn : v * cs + u * sn;
        } else {
            y = to_f(src[c]);
            if (c < ncols) y = y * inv * to_f(k_norm_w[c]);
        }
        dst[c] = from_f<T>(pos >= 0 ? y : 0.0f);
    }
}

// ---- the general kernel: any sizes and strides, any dtype, 32-bit arithmetic throughout (float32 models, decoding, short
// portions).  A block of SA_WARPS warps per (token, query head); the warps take the visible keys in turns of 32, each with its
// own running maximum, sum and weighted values; the warps' partial results are merged in shared memory in warp order.
constexpr int SA_WARPS = 8;
constexpr int SA_VCOLS = 16;                                // value columns a lane owns per pass (columns lane, lane + 32, ...)

template <typename T>
__device__ __forceinline__ float dot_strided(const float* __restrict__ qs, const T* __restrict__ kr, int dim, bool aligned) {
    if (aligned) return dot_row(qs, kr, dim);
    float s = 0.0f;
    for (int d = 0; d < dim; ++d) s += qs[d] * to_f(kr[d]);
    return s;
}

template <typename T>
__global__ void __launch_bounds__(SA_WARPS * 32) softmax_attention_kernel(
        const T* __restrict__ q, long q_ld, long q_hs, const T* __restrict__ k, long k_bs, long k_ps, long k_hs, const T* __restrict__ v, long v_bs, long v_ps,
        long v_hs, int B, int S, int heads, int kv_heads, int dim, int vdim, int held, int shift, const int32_t* __restrict__ pad, int window, int chunk,
        float scale, float softcap, const T* __restrict__ sink, T* __restrict__ out, long ld_out, int out_col, const int32_t* __restrict__ dyn, int aligned) {
    extern __shared__ __align__(16) float sa_sh[];          // q [dim rounded up to 4], warp maxima, warp sums, partial values
    const int dim4 = (dim + 3) & ~3;
    float* qs = sa_sh;
    float* wm = sa_sh + dim4;
    float* wl = wm + SA_WARPS;
    float* part = wl + SA_WARPS;                            // [SA_WARPS][SA_VCOLS * 32]
    if (dyn) held = dyn[0];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = blockIdx.x;
    const long n = item / heads;
    const int h = (int)(item - n * heads);
    const int b = (int)(n / S), t = (int)(n - (long)b * S);
    const int g = h / (heads / kv_heads);
    const int c = held + t;                                 // the query's own storage index
    T* dst = out + n * ld_out + out_col + (long)h * vdim;
    const int first_real = pad[b] - shift;
    if (c < first_real) {
        for (int col = threadIdx.x; col < vdim; col += blockDim.x) dst[col] = from_f<T>(0.0f);
        return;
    }
    const int lo = visible_from(c, first_real, window, chunk);
    const T* qsrc = q + n * q_ld + h * q_hs;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) qs[d] = to_f(qsrc[d]);
    __syncthreads();
    const T* kbase = k + b * k_bs + g * k_hs;
    const T* vbase = v + b * v_bs + g * v_hs;
    for (int col0 = 0; col0 < vdim; col0 += SA_VCOLS * 32) {
        float m = -INFINITY, l = 0.0f;
        float acc[SA_VCOLS];
#pragma unroll
        for (int i = 0; i < SA_VCOLS; ++i) acc[i] = 0.0f;
        for (int j0 = lo + 32 * wid; j0 <= c; j0 += 32 * SA_WARPS) {
            const int j = j0 + lane;
            float s = -INFINITY;
            if (j <= c) {
                s = dot_strided(qs, kbase + j * k_ps, dim, aligned != 0) * scale;
                if (softcap > 0.0f) s = softcap * tanhf(s / softcap);
            }
            const float m_new = fmaxf(m, warp_max(s));      // finite: key j0 is visible
            const float corr = expf(m - m_new);             // 0 on the first turn (m = -inf)
            const float p = j <= c ? expf(s - m_new) : 0.0f;
            l = l * corr + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int i = 0; i < SA_VCOLS; ++i) acc[i] *= corr;
            const int nk = c - j0 + 1 < 32 ? c - j0 + 1 : 32;
            for (int jj = 0; jj < nk; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const T* vr = vbase + (j0 + jj) * v_ps + col0;
#pragma unroll
                for (int i = 0; i < SA_VCOLS; ++i) {
                    const int col = lane + 32 * i;
                    if (col0 + col < vdim) acc[i] += pj * to_f(vr[col]);
                }
            }
        }
        if (lane == 0) { wm[wid] = m; wl[wid] = l; }
#pragma unroll
        for (int i = 0; i < SA_VCOLS; ++i) part[(wid * SA_VCOLS + i) * 32 + lane] = acc[i];
        __syncthreads();
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < SA_WARPS; ++w) big = fmaxf(big, wm[w]);
        float f[SA_WARPS], total = 0.0f;
#pragma unroll
        for (int w = 0; w < SA_WARPS; ++w) { f[w] = wm[w] == -INFINITY ? 0.0f : expf(wm[w] - big); total += wl[w] * f[w]; }
        if (sink) total += expf(to_f(sink[h]) - big);       // a sink far above every score: the sum overflows and the output is 0, its limit
        for (int e = threadIdx.x; e < SA_VCOLS * 32; e += blockDim.x) {
            const int col = col0 + e;                       // e = i * 32 + lane, column = col0 + lane + 32 i
            if (col < vdim) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < SA_WARPS; ++w) sum += part[w * SA_VCOLS * 32 + e] * f[w];
                dst[col] = from_f<T>(sum / total);
            }
        }
        __syncthreads();
    }
}

// ---- many new tokens of a 16-bit model: both products on the tensor cores (mma.sync m16n8k16, 32-bit accumulators).
// A block of 4 warps takes 64 consecutive query tokens of one head (16 rows a warp, queries as A fragments in registers) and
// walks the keys they can see 32 at a time: K and V tiles staged in shared memory (rows padded by 16 bytes: conflict-free
// fragment reads and transposing ldmatrix), S = Q K^T, then per row the running maximum and sum of the softmax in 32-bit
// floats, P = exp(S - max) with everything a row cannot see set to zero, O = O * correction + P V.  P goes to the tensor cores
// as the sum of two 16-bit numbers (its rounding and the rounding's remainder): the weights keep ~16 bits of mantissa.
template <typename T> struct SaMma;
template <> struct SaMma<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct SaMma<__half> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

constexpr int SA_ROWS = 64, SA_KEYS = 32;

// cap * tanh(s / cap) with the hardware exponential: tanh(y) = 1 - 2 / (e^2y + 1), exact at both ends (cap <= 0: s itself)
__device__ __forceinline__ float fast_cap(float s, float cap, float inv_cap) {
    if (cap <= 0.0f) return s;
    return cap * (1.0f - __fdividef(2.0f, __expf(2.0f * s * inv_cap) + 1.0f));
}

template <typename T, int KDMAX, int NDMAX>                // dim <= 16 KDMAX, vdim <= 8 NDMAX; both multiples of 16
__global__ void __launch_bounds__(128) softmax_attention_tc_kernel(
        const T* __restrict__ q, long q_ld, long q_hs, const T* __restrict__ k, long k_bs, long k_ps, long k_hs, const T* __restrict__ v, long v_bs, long v_ps,
        long v_hs, int B, int S, int heads, int kv_heads, int dim, int vdim, int held, int shift, const int32_t* __restrict__ pad, int window, int chunk,
        float scale, float softcap, const T* __restrict__ sink, T* __restrict__ out, long ld_out, int out_col) {
    extern __shared__ __align__(16) unsigned char sa_tc_sh[];
    const int kstride = dim + 8, vstride = vdim + 8;        // elements
    T* Ks = reinterpret_cast<T*>(sa_tc_sh);                 // two stages of [SA_KEYS][kstride] keys + [SA_KEYS][vstride] values
    // the last query tiles first: they see the most keys
    const int b = blockIdx.z, h = blockIdx.y, t0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * SA_ROWS;
    const int g = h / (heads / kv_heads);
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31, gr = lane >> 2, tq = lane & 3;
    const int kdn = dim >> 4, ndn = vdim >> 3;
    const int first_real = pad[b] - shift;
    const int t_last = (t0 + SA_ROWS - 1 < S - 1) ? t0 + SA_ROWS - 1 : S - 1;
    const int c_hi = held + t_last;                         // newest key this block can see
    const int j_start = visible_from(held + t0, first_real, window, chunk);
    const int r0 = t0 + wid * 16;                           // this warp's rows
    const int tr[2] = {r0 + gr, r0 + gr + 8};
    int row_c[2], row_lo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        row_c[i] = held + tr[i];
        row_lo[i] = visible_from(row_c[i], first_real, window, chunk);
        if (tr[i] >= S || row_c[i] < first_real) { row_c[i] = -1; row_lo[i] = 0; }      // nothing visible
    }
    const int warp_hi = held + ((r0 + 15 < S - 1) ? r0 + 15 : S - 1);
    const int warp_lo = visible_from(held + r0, first_real, window, chunk);
    uint32_t qa[KDMAX][4];
#pragma unroll
    for (int kd = 0; kd < KDMAX; ++kd) {
#pragma unroll
        for (int i = 0; i < 4; ++i) qa[kd][i] = 0u;
        if (kd < kdn) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (tr[i] < S) {
                    const T* src = q + ((long)b * S + tr[i]) * q_ld + h * q_hs + kd * 16 + 2 * tq;
                    qa[kd][i] = *reinterpret_cast<const uint32_t*>(src);
                    qa[kd][2 + i] = *reinterpret_cast<const uint32_t*>(src + 8);
                }
            }
        }
    }
    float oacc[NDMAX][4];
#pragma unroll
    for (int nd = 0; nd < NDMAX; ++nd)
#pragma unroll
        for (int i = 0; i < 4; ++i) oacc[nd][i] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};      // l: this lane's share of the row's sum
    const T* kbase = k + b * k_bs + g * k_hs;
    const T* vbase = v + b * v_bs + g * v_hs;
    const int kchunks = dim >> 3, vchunks = vdim >> 3;      // 16-byte pieces per row
    const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;
    const float sinkv = sink ? to_f(sink[h]) : -INFINITY;

    // two stages of K / V tiles: the next tile's copies (cp.async, 16 bytes each) are in flight while this one is multiplied
    auto load_tile = [&](int stage, int jt) {
        T* kd_ = Ks + stage * SA_KEYS * (kstride + vstride);
        T* vd_ = kd_ + SA_KEYS * kstride;
        for (int id = tid; id < SA_KEYS * kchunks; id += 128) {
            int r = id / kchunks, cch = id - r * kchunks;
            int j = jt + r <= c_hi ? jt + r : c_hi;         // rows past the end repeat the last one (their weights are zero)
            uint32_t dst = (uint32_t)__cvta_generic_to_shared(kd_ + r * kstride + cch * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(dst), "l"(kbase + j * k_ps + cch * 8));
        }
        for (int id = tid; id < SA_KEYS * vchunks; id += 128) {
            int r = id / vchunks, cch = id - r * vchunks;
            int j = jt + r <= c_hi ? jt + r : c_hi;
            uint32_t dst = (uint32_t)__cvta_generic_to_shared(vd_ + r * vstride + cch * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(dst), "l"(vbase + j * v_ps + cch * 8));
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    if (j_start <= c_hi) load_tile(0, j_start);
    int stage = 0;
    for (int jt = j_start; jt <= c_hi; jt += SA_KEYS, stage ^= 1) {
        if (jt + SA_KEYS <= c_hi) {
            load_tile(stage ^ 1, jt + SA_KEYS);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();                                    // this tile has arrived for every thread
        const T* Kt = Ks + stage * SA_KEYS * (kstride + vstride);
        const T* Vt = Kt + SA_KEYS * kstride;
        if (!(jt > warp_hi || jt + SA_KEYS - 1 < warp_lo)) {               // some row of this warp sees the tile
            float sc[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) sc[nt][i] = 0.0f;
                const T* krow = Kt + (nt * 8 + gr) * kstride + 2 * tq;
#pragma unroll
                for (int kd = 0; kd < KDMAX; ++kd) {
                    if (kd < kdn) {
                        uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + kd * 16);
                        uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + kd * 16 + 8);
                        SaMma<T>::mma(sc[nt], qa[kd], b0, b1);
                    }
                }
            }
            // scores -> masked, scaled; the rows' new maxima
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j = jt + nt * 8 + 2 * tq + (i & 1);
                    const int r = i >> 1;
                    const float s = (j >= row_lo[r] && j <= row_c[r]) ? fast_cap(sc[nt][i] * scale, softcap, inv_cap) : -INFINITY;
                    sc[nt][i] = s;
                    tmax[r] = fmaxf(tmax[r], s);
                }
            }
            float corr[2], m_new[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
                m_new[r] = fmaxf(m_run[r], tmax[r]);
                corr[r] = m_new[r] == -INFINITY ? 1.0f : __expf(m_run[r] - m_new[r]);
                m_run[r] = m_new[r];
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int nd = 0; nd < NDMAX; ++nd) {
                oacc[nd][0] *= corr[0]; oacc[nd][1] *= corr[0];
                oacc[nd][2] *= corr[1]; oacc[nd][3] *= corr[1];
            }
            uint32_t ph[2][4], pl[2][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                float p[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = i >> 1;
                    p[i] = sc[nt][i] == -INFINITY ? 0.0f : __expf(sc[nt][i] - m_new[r]);
                    l_run[r] += p[i];
                }
                const int ks = nt >> 1, half = nt & 1;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    uint32_t hi = SaMma<T>::pack(p[2 * r], p[2 * r + 1]);
                    float2 back = SaMma<T>::unpack(hi);
                    ph[ks][2 * half + r] = hi;
                    pl[ks][2 * half + r] = SaMma<T>::pack(p[2 * r] - back.x, p[2 * r + 1] - back.y);
                }
            }
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
                for (int np = 0; np < NDMAX / 2; ++np) {
                    if (2 * np < ndn) {
                        uint32_t v0, v1, v2, v3;
                        const T* vaddr = Vt + (ks * 16 + (lane & 15)) * vstride + np * 16 + ((lane >> 4) << 3);
                        uint32_t sa = (uint32_t)__cvta_generic_to_shared(vaddr);
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                                     : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(sa));
                        SaMma<T>::mma(oacc[2 * np], ph[ks], v0, v1);
                        SaMma<T>::mma(oacc[2 * np], pl[ks], v0, v1);
                        SaMma<T>::mma(oacc[2 * np + 1], ph[ks], v2, v3);
                        SaMma<T>::mma(oacc[2 * np + 1], pl[ks], v2, v3);
                    }
                }
            }
        }
        __syncthreads();                                    // the tile has been consumed: its stage may be overwritten
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float l = l_run[i];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (l > 0.0f && sink) l += __expf(sinkv - m_run[i]);                 // overflow = a sink far above every score: output 0
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        if (tr[i] < S) {
            T* dst = out + ((long)b * S + tr[i]) * ld_out + out_col + (long)h * vdim + 2 * tq;
#pragma unroll
            for (int nd = 0; nd < NDMAX; ++nd) {
                if (nd < ndn) {
                    dst[nd * 8] = from_f<T>(oacc[nd][2 * i] * inv);
                    dst[nd * 8 + 1] = from_f<T>(oacc[nd][2 * i + 1] * inv);
                }
            }
        }
    }
}

// ---- few new tokens of a 16-bit model whose query heads share key / value heads (one shared head in the extreme: a latent
// cache read as key AND value): the 16 rows of an MMA tile are (token, head) pairs of one group, so ONE pass over the keys
// serves them all.  grid (key splits, 16-row tiles x kv heads, batch); a block of 8 warps walks its range of keys 64 at a
// time: the tile of keys in shared memory (once, when keys and values are the same tensor), S = Q K^T with each warp taking 8
// keys, the scaled and masked scores through shared memory, then every warp forms the rows' running maxima and the weights
// (as the sum of two 16-bit numbers, like the prompt kernel) and multiplies them into ITS 1/8 of the value columns.  Each
// block leaves (max, sum, weighted values) of its key range in the workspace; shared_head_merge_kernel adds the ranges up.
constexpr int SH_KEYS = 64, SH_SSTRIDE = 72, SH_MIN_CHUNK = 64, SH_MAX_SPLITS = 32;

template <typename T, int NT, bool SAME>                   // vdim = 64 NT (each warp owns 8 NT value columns)
__global__ void __launch_bounds__(256) shared_head_attention_kernel(
        const T* __restrict__ q, long q_ld, long q_hs, const T* __restrict__ k, long k_bs, long k_ps, long k_hs, const T* __restrict__ v, long v_bs, long v_ps,
        long v_hs, int B, int S, int heads, int kv_heads, int dim, int held, int shift, const int32_t* __restrict__ pad, int window, int chunk, float scale,
        float softcap, float* __restrict__ ws, int splits, int tiles, const int32_t* __restrict__ dyn) {
    constexpr int vdim = 64 * NT;
    extern __shared__ __align__(16) unsigned char sh_raw[];
    const int kstride = dim + 8, vstride = vdim + 8;
    const int stage_elems = SH_KEYS * kstride + (SAME ? 0 : SH_KEYS * vstride);
    T* Qs = reinterpret_cast<T*>(sh_raw);                   // [16][kstride]
    T* Kst = Qs + 16 * kstride;                             // two stages of [SH_KEYS][kstride] keys (+ [SH_KEYS][vstride] values)
    float* Ss = reinterpret_cast<float*>(Kst + 2 * stage_elems);                                         // [16][SH_SSTRIDE]
    int* row_c = reinterpret_cast<int*>(Ss + 16 * SH_SSTRIDE);                                           // [16] newest visible key, -1: none
    int* row_lo = row_c + 16;                                                                            // [16] oldest visible key
    if (dyn) held = dyn[0];
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31, gr = lane >> 2, tq = lane & 3;
    const int split = blockIdx.x, b = blockIdx.z;
    const int g = blockIdx.y / tiles, tile = blockIdx.y - g * tiles;
    const int gs = heads / kv_heads, n_rows = S * gs;
    const int first_real = pad[b] - shift;
    if (tid < 16) {
        const int r = tile * 16 + tid;
        int c = -1, lo = 0;
        if (r < n_rows) {
            c = held + r / gs;
            lo = visible_from(c, first_real, window, chunk);
            if (c < first_real) c = -1;
        }
        row_c[tid] = c;
        row_lo[tid] = lo;
    }
    __syncthreads();
    int lo_all = 0x7fffffff, hi_all = -1;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        if (row_c[i] >= 0) { lo_all = min(lo_all, row_lo[i]); hi_all = max(hi_all, row_c[i]); }
    }
    const int my_c[2] = {row_c[gr], row_c[gr + 8]}, my_lo[2] = {row_lo[gr], row_lo[gr + 8]};
    // this block's range of keys
    int j_lo = 0, j_hi = -1;
    if (hi_all >= 0) {
        const int nkeys = hi_all - lo_all + 1;
        int chunk = ((nkeys + splits - 1) / splits + SH_KEYS - 1) / SH_KEYS * SH_KEYS;
        if (chunk < SH_MIN_CHUNK) chunk = SH_MIN_CHUNK;
        j_lo = lo_all + split * chunk;
        j_hi = min(hi_all, j_lo + chunk - 1);
    }
    float oacc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) oacc[nt][i] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const T* kbase = k + b * k_bs + g * k_hs;
    const T* vbase = v + b * v_bs + g * v_hs;
    const int kchunks = dim >> 3, vchunks = vdim >> 3, kdn = dim >> 4;
    const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;

    // two stages of key (and value) tiles: the next tile's copies (cp.async, 16 bytes each) fly while this one is multiplied
    auto load_tile = [&](int stage, int jt) {
        T* kd_ = Kst + stage * stage_elems;
        for (int id = tid; id < SH_KEYS * kchunks; id += 256) {
            const int r = id / kchunks, cch = id - r * kchunks;
            const int j = jt + r <= j_hi ? jt + r : j_hi;   // rows past the end repeat the last one (their weights are zero)
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(kd_ + r * kstride + cch * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(dst), "l"(kbase + j * k_ps + cch * 8));
        }
        if (!SAME) {
            T* vd_ = kd_ + SH_KEYS * kstride;
            for (int id = tid; id < SH_KEYS * vchunks; id += 256) {
                const int r = id / vchunks, cch = id - r * vchunks;
                const int j = jt + r <= j_hi ? jt + r : j_hi;
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(vd_ + r * vstride + cch * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(dst), "l"(vbase + j * v_ps + cch * 8));
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    if (j_lo <= j_hi) load_tile(0, j_lo);
    {   // the queries of this tile's rows, zeros for rows that do not exist (while the first keys are on their way)
        const int qchunks = dim >> 3;
        for (int id = tid; id < 16 * qchunks; id += 256) {
            const int i = id / qchunks, cch = id - i * qchunks;
            const int r = tile * 16 + i;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (r < n_rows) val = *reinterpret_cast<const uint4*>(q + ((long)b * S + r / gs) * q_ld + (g * gs + r % gs) * q_hs + cch * 8);
            *reinterpret_cast<uint4*>(Qs + i * kstride + cch * 8) = val;
        }
    }
    int stage = 0;
    for (int jt = j_lo; jt <= j_hi; jt += SH_KEYS, stage ^= 1) {
        if (jt + SH_KEYS <= j_hi) {
            load_tile(stage ^ 1, jt + SH_KEYS);            // its stage was consumed before the barrier that ended the last turn
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();                                    // this tile (and, the first time, the queries) is there for every thread
        const T* Ks = Kst + stage * stage_elems;
        const T* Vs = SAME ? Ks : Ks + SH_KEYS * kstride;
        {   // scores of keys 8 wid .. 8 wid + 7 for the 16 rows
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const T* qrow = Qs + gr * kstride + 2 * tq;
            const T* krow = Ks + (wid * 8 + gr) * kstride + 2 * tq;
            for (int kd = 0; kd < kdn; ++kd) {
                uint32_t a[4];
                a[0] = *reinterpret_cast<const uint32_t*>(qrow + kd * 16);
                a[1] = *reinterpret_cast<const uint32_t*>(qrow + 8 * kstride + kd * 16);
                a[2] = *reinterpret_cast<const uint32_t*>(qrow + kd * 16 + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(qrow + 8 * kstride + kd * 16 + 8);
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + kd * 16);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + kd * 16 + 8);
                SaMma<T>::mma(sc, a, b0, b1);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float2 out;
                const int j = jt + wid * 8 + 2 * tq;
                out.x = (j >= my_lo[r] && j <= my_c[r] && j <= j_hi) ? fast_cap(sc[2 * r] * scale, softcap, inv_cap) : -INFINITY;
                out.y = (j + 1 >= my_lo[r] && j + 1 <= my_c[r] && j + 1 <= j_hi) ? fast_cap(sc[2 * r + 1] * scale, softcap, inv_cap) : -INFINITY;
                *reinterpret_cast<float2*>(Ss + (gr + 8 * r) * SH_SSTRIDE + wid * 8 + 2 * tq) = out;
            }
        }
        __syncthreads();
        // every warp: the rows' maxima and weights over the 64 keys (a lane holds the 16 keys of its A fragments per row)
        float2 sv[2][4][2];
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const float2 x = *reinterpret_cast<const float2*>(Ss + (gr + 8 * r) * SH_SSTRIDE + ks * 16 + half * 8 + 2 * tq);
                    sv[r][ks][half] = x;
                    tmax[r] = fmaxf(tmax[r], fmaxf(x.x, x.y));
                }
        float corr[2], m_new[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
            m_new[r] = fmaxf(m_run[r], tmax[r]);
            corr[r] = m_new[r] == -INFINITY ? 1.0f : __expf(m_run[r] - m_new[r]);
            m_run[r] = m_new[r];
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            oacc[nt][0] *= corr[0]; oacc[nt][1] *= corr[0];
            oacc[nt][2] *= corr[1]; oacc[nt][3] *= corr[1];
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const float2 x = sv[r][ks][half];
                    const float p0 = x.x == -INFINITY ? 0.0f : __expf(x.x - m_new[r]);
                    const float p1 = x.y == -INFINITY ? 0.0f : __expf(x.y - m_new[r]);
                    l_run[r] += p0 + p1;
                    const uint32_t hi = SaMma<T>::pack(p0, p1);
                    const float2 back = SaMma<T>::unpack(hi);
                    ph[2 * half + r] = hi;
                    pl[2 * half + r] = SaMma<T>::pack(p0 - back.x, p1 - back.y);
                }
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t v0, v1, v2, v3;
                const T* vaddr = Vs + (ks * 16 + (lane & 15)) * (SAME ? kstride : vstride) + wid * (8 * NT) + np * 16 + ((lane >> 4) << 3);
                const uint32_t sa = (uint32_t)__cvta_generic_to_shared(vaddr);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(sa));
                SaMma<T>::mma(oacc[2 * np], ph, v0, v1);
                SaMma<T>::mma(oacc[2 * np], pl, v0, v1);
                SaMma<T>::mma(oacc[2 * np + 1], ph, v2, v3);
                SaMma<T>::mma(oacc[2 * np + 1], pl, v2, v3);
            }
        }
        __syncthreads();                                    // tile and scores consumed: the next turn overwrites this stage
    }
    // this range's share: per row the maximum, the sum, and the weighted values
    float* base = ws + (((long)b * gridDim.y + blockIdx.y) * splits + split) * (16L * (vdim + 2));
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = l_run[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        float* rowp = base + (gr + 8 * r) * (long)(vdim + 2);
        if (wid == 0 && tq == 0) { rowp[0] = m_run[r]; rowp[1] = l; }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            *reinterpret_cast<float2*>(rowp + 2 + wid * (8 * NT) + nt * 8 + 2 * tq) = make_float2(oacc[nt][2 * r], oacc[nt][2 * r + 1]);
    }
}

// grid (16 x 16-row tiles x kv heads, batch): one block per row adds up the key ranges' shares.  Warp 0 turns the ranges'
// maxima into factors; then every thread owns two neighbouring columns and reads them from all ranges (independent loads).
template <typename T>
__global__ void __launch_bounds__(256) shared_head_merge_kernel(const float* __restrict__ ws, int S, int heads, int kv_heads, int vdim, int splits,
                                                                int tiles, const T* __restrict__ sink, T* __restrict__ out, long ld_out, int out_col) {
    __shared__ float factor[SH_MAX_SPLITS];
    __shared__ float inv_total;
    const int y = blockIdx.x >> 4, i = blockIdx.x & 15, lane = threadIdx.x & 31;
    const int b = blockIdx.y, g = y / tiles, tile = y - g * tiles;
    const int gs = heads / kv_heads;
    const int r = tile * 16 + i;
    if (r >= S * gs) return;
    const long sstride = 16L * (vdim + 2);
    const float* base = ws + ((long)b * (gridDim.x >> 4) + y) * splits * sstride + i * (long)(vdim + 2);
    if (threadIdx.x < 32) {
        const float m = lane < splits ? base[lane * sstride] : -INFINITY;
        const float l = lane < splits ? base[lane * sstride + 1] : 0.0f;
        const float big = warp_max(m);
        const float f = m == -INFINITY ? 0.0f : __expf(m - big);
        float total = warp_sum(l * f);
        if (sink && total > 0.0f) total += __expf(to_f(sink[g * gs + r % gs]) - big);
        factor[lane] = f;
        if (lane == 0) inv_total = total > 0.0f ? 1.0f / total : 0.0f;
    }
    __syncthreads();
    T* dst = out + ((long)b * S + r / gs) * ld_out + out_col + (long)(g * gs + r % gs) * vdim;
    for (int col = 2 * threadIdx.x; col < vdim; col += 512) {
        float sx = 0.0f, sy = 0.0f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            if (factor[s] == 0.0f) continue;                // an empty range (the same for the whole block)
            const float2 o = *reinterpret_cast<const float2*>(base + s * sstride + 2 + col);
            sx += o.x * factor[s];
            sy += o.y * factor[s];
        }
        dst[col] = from_f<T>(sx * inv_total);
        dst[col + 1] = from_f<T>(sy * inv_total);
    }
}

static int shared_head_splits(int B, int S, int heads, int kv_heads) {
    const int tiles = (S * (heads / kv_heads) + 15) / 16;
    long blocks = (long)B * kv_heads * tiles;
    long s = (148 + blocks - 1) / blocks;                   // one block per SM (two stages of key tiles fill its shared memory)
    return (int)(s < 1 ? 1 : (s > SH_MAX_SPLITS ? SH_MAX_SPLITS : s));
}

static bool shared_head_ok(int dtype, int S, int heads, int kv_heads, int dim, int vdim) {
    return dtype != 0 && kv_heads >= 1 && heads % kv_heads == 0 && heads / kv_heads >= 4 && S <= 16 && dim % 16 == 0 && dim <= 1024 &&
           (vdim == 128 || vdim == 256 || vdim == 512);
}

static size_t shared_head_smem(int dim, int vdim, bool same) {
    return (size_t)(16 + 2 * SH_KEYS) * (dim + 8) * 2 + (same ? 0 : 2 * (size_t)SH_KEYS * (vdim + 8) * 2) + 16 * SH_SSTRIDE * sizeof(float) +
           32 * sizeof(int);
}

template <typename T, int NT>
static int launch_shared_head(const void* q, long q_ld, long q_hs, const void* k, long k_bs, long k_ps, long k_hs, const void* v, long v_bs, long v_ps, long v_hs,
                              int B, int S, int heads, int kv_heads, int dim, int held, int shift, const int32_t* pad, int window, int chunk, float scale,
                              float softcap, const void* sink, void* out, long ld_out, int out_col, const int32_t* dyn, float* ws, cudaStream_t stream) {
    const int vdim = 64 * NT;
    const int tiles = (S * (heads / kv_heads) + 15) / 16, splits = shared_head_splits(B, S, heads, kv_heads);
    const bool same = k == v && k_bs == v_bs && k_ps == v_ps && k_hs == v_hs && dim >= vdim;     // the values are the keys' first channels
    const size_t smem = shared_head_smem(dim, vdim, same);
    dim3 grid(splits, tiles * kv_heads, B);
    cudaError_t err;
    if (same) {
        auto fn = shared_head_attention_kernel<T, NT, true>;
        if ((err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)err;
        fn<<<grid, 256, smem, stream>>>((const T*)q, q_ld, q_hs, (const T*)k, k_bs, k_ps, k_hs, (const T*)v, v_bs, v_ps, v_hs, B, S, heads, kv_heads, dim, held,
                                        shift, pad, window, chunk, scale, softcap, ws, splits, tiles, dyn);
    } else {
        auto fn = shared_head_attention_kernel<T, NT, false>;
        if ((err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)err;
        fn<<<grid, 256, smem, stream>>>((const T*)q, q_ld, q_hs, (const T*)k, k_bs, k_ps, k_hs, (const T*)v, v_bs, v_ps, v_hs, B, S, heads, kv_heads, dim, held,
                                        shift, pad, window, chunk, scale, softcap, ws, splits, tiles, dyn);
    }
    if ((err = cudaGetLastError()) != cudaSuccess) return (int)err;
    shared_head_merge_kernel<T><<<dim3(16 * tiles * kv_heads, B), 256, 0, stream>>>(ws, S, heads, kv_heads, vdim, splits, tiles, (const T*)sink, (T*)out, ld_out, out_col);
    return mixers_status();
}

#define SA_TC_PARAMS const void* q, long q_ld, long q_hs, const void* k, long k_bs, long k_ps, long k_hs, const void* v, long v_bs, long v_ps, long v_hs, \
    int B, int S, int heads, int kv_heads, int dim, int vdim, int held, int shift, const int32_t* pad, int window, int chunk, float scale, float softcap,  \
    const void* sink, void* out, long ld_out, int out_col, cudaStream_t stream
#define SA_TC_ARGS q, q_ld, q_hs, k, k_bs, k_ps, k_hs, v, v_bs, v_ps, v_hs, B, S, heads, kv_heads, dim, vdim, held, shift, pad, window, chunk, scale, softcap, \
    sink, out, ld_out, out_col, stream

template <typename T, int KDMAX, int NDMAX>
static int launch_softmax_tc(SA_TC_PARAMS) {
    size_t smem = 2 * (size_t)SA_KEYS * (dim + 8 + vdim + 8) * sizeof(T);
    dim3 grid((S + SA_ROWS - 1) / SA_ROWS, heads, B);
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(softmax_attention_tc_kernel<T, KDMAX, NDMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    softmax_attention_tc_kernel<T, KDMAX, NDMAX><<<grid, 128, smem, stream>>>(
        (const T*)q, q_ld, q_hs, (const T*)k, k_bs, k_ps, k_hs, (const T*)v, v_bs, v_ps, v_hs, B, S, heads, kv_heads, dim, vdim, held, shift, pad, window, chunk,
        scale, softcap, (const T*)sink, (T*)out, ld_out, out_col);
    return mixers_status();
}

template <typename T>
static int softmax_tc(SA_TC_PARAMS) {
    if (dim <= 64 && vdim <= 64) return launch_softmax_tc<T, 4, 8>(SA_TC_ARGS);
    if (dim <= 128 && vdim <= 128) return launch_softmax_tc<T, 8, 16>(SA_TC_ARGS);
    return launch_softmax_tc<T, 16, 32>(SA_TC_ARGS);
}

extern "C" int mixers_latent_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int q_rank, const void* q_w, int off_c,
                                     int kv_rank, const void* c_w, float eps, void* cq_out, void* store, int cap, int held, int shift,
                                     const int32_t* pad, const int32_t* dyn, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (held + S > cap) return (int)cudaErrorInvalidValue;
    MIXERS_DISPATCH(dtype, latent_prepare_kernel<T><<<(unsigned)(2L * B * S), LP_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)proj, B, S, ld, off_q, q_rank, (const T*)q_w, off_c, kv_rank, (const T*)c_w, eps, (T*)cq_out, (T*)store, cap, held, shift, pad, dyn));
    return mixers_status();
}

extern "C" int mixers_wide_qkv_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads,
                                       int dim, int vdim, const void* q_w, const void* k_w, float eps, const void* v_other, long ld_other,
                                       const void* blend, void* q_out, void* k_store, void* v_store, int cap, int held, int shift,
                                       const int32_t* pad, const int32_t* dyn, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (held + S > cap || (v_other && !blend)) return (int)cudaErrorInvalidValue;
    int threads = 128;
    if ((long)B * S <= QP_FEW_TOKENS)
        while (threads < 1024 && threads * QP_MAXC < heads * dim) threads <<= 1;
#define QP_LAUNCH(TH) MIXERS_DISPATCH(dtype, wide_qkv_prepare_kernel<T, TH><<<(unsigned)(3L * B * S), TH, 0, (cudaStream_t)stream>>>(               \
        (const T*)proj, B, S, ld, off_q, off_k, off_v, heads, kv_heads, dim, vdim, (const T*)q_w, (const T*)k_w, eps, (const T*)v_other, ld_other, \
        (const T*)blend, (T*)q_out, (T*)k_store, (T*)v_store, cap, held, shift, pad, dyn))
    if (threads == 128) QP_LAUNCH(128);
    else if (threads == 256) QP_LAUNCH(256);
    else if (threads == 512) QP_LAUNCH(512);
    else QP_LAUNCH(1024);
#undef QP_LAUNCH
    return mixers_status();
}

extern "C" int mixers_rope_qk_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads,
                                      int q_dim, int k_dim, int vdim, int q_rot_off, int k_rot_off, int rot_dims, const double* inv_freq, float amp,
                                      const void* k_norm_w, int k_norm_cols, float eps, void* q_out, void* k_store, long k_bs, long k_ps,
                                      long k_hs, void* v_store, long v_bs, long v_ps, long v_hs, int held, int shift, const int32_t* pad,
                                      const int32_t* dyn, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (rot_dims < 0 || (rot_dims & 1) || q_rot_off < 0 || k_rot_off < 0 || q_rot_off + rot_dims > q_dim || k_rot_off + rot_dims > k_dim ||
        kv_heads < 1 || heads < 1 || (rot_dims > 0 && !inv_freq) || (k_norm_w && (k_norm_cols < 1 || k_norm_cols > k_rot_off)) || (vdim > 0 && !v_store))
        return (int)cudaErrorInvalidValue;
    const long warps = (long)B * S * (heads + kv_heads + (vdim > 0 ? kv_heads : 0));
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    MIXERS_DISPATCH(dtype, rope_qk_prepare_kernel<T><<<blocks, 128, 0, (cudaStream_t)stream>>>(
        (const T*)proj, B, S, ld, off_q, off_k, off_v, heads, kv_heads, q_dim, k_dim, vdim, q_rot_off, k_rot_off, rot_dims, inv_freq, amp,
        (const T*)k_norm_w, k_norm_cols, eps, (T*)q_out, (T*)k_store, k_bs, k_ps, k_hs, (T*)v_store, v_bs, v_ps, v_hs, held, shift, pad, dyn));
    return mixers_status();
}

extern "C" int mixers_softmax_attention(int dtype, const void* q, long q_ld, long q_hs, const void* k, long k_bs, long k_ps, long k_hs, const void* v,
                                        long v_bs, long v_ps, long v_hs, int B, int S, int heads, int kv_heads, int dim, int vdim, int held,
                                        int shift, const int32_t* pad, int window, int chunk, float scale, float softcap, const void* sink, void* out,
                                        long ld_out, int out_col, const int32_t* dyn, int allow_tensor_cores, float* ws, mixers_stream_t stream_) {
    if (B <= 0 || S <= 0) return 0;
    cudaStream_t stream = (cudaStream_t)stream_;
    const int dim4 = (dim + 3) & ~3;
    size_t smem = ((size_t)dim4 + 2 * SA_WARPS + SA_WARPS * SA_VCOLS * 32) * sizeof(float);
    if (window < 0 || chunk < 0 || kv_heads < 1 || heads % kv_heads != 0 || smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const size_t esz = dtype == 0 ? 4 : 2;
    auto mult8 = [](long s) { return (s & 7) == 0; };
    const bool rows16 = esz == 2 && mult8(k_bs) && mult8(k_ps) && mult8(k_hs) && mult8(v_bs) && mult8(v_ps) && mult8(v_hs) &&
                        ((uintptr_t)k & 15) == 0 && ((uintptr_t)v & 15) == 0 && (dim & 7) == 0;
    const bool same_kv = k == v && k_bs == v_bs && k_ps == v_ps && k_hs == v_hs && dim >= vdim;
    if (allow_tensor_cores && ws && rows16 && shared_head_ok(dtype, S, heads, kv_heads, dim, vdim) && (q_ld & 7) == 0 && (q_hs & 7) == 0 && ((uintptr_t)q & 15) == 0 &&
        (ld_out & 1) == 0 && (out_col & 1) == 0 && shared_head_smem(dim, vdim, same_kv) <= 227 * 1024) {
#define SH_ARGS q, q_ld, q_hs, k, k_bs, k_ps, k_hs, v, v_bs, v_ps, v_hs, B, S, heads, kv_heads, dim, held, shift, pad, window, chunk, scale, softcap, sink, out, ld_out, out_col, dyn, ws, stream
        if (dtype == 1) return vdim == 128 ? launch_shared_head<__nv_bfloat16, 2>(SH_ARGS) : vdim == 256 ? launch_shared_head<__nv_bfloat16, 4>(SH_ARGS)
                                                                                                       : launch_shared_head<__nv_bfloat16, 8>(SH_ARGS);
        return vdim == 128 ? launch_shared_head<__half, 2>(SH_ARGS) : vdim == 256 ? launch_shared_head<__half, 4>(SH_ARGS)
                                                                                  : launch_shared_head<__half, 8>(SH_ARGS);
#undef SH_ARGS
    }
    if (allow_tensor_cores && dtype != 0 && !dyn && S >= 16 && rows16 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 256 && vdim <= 256 &&
        (q_ld & 1) == 0 && (q_hs & 1) == 0 && ((uintptr_t)q & 3) == 0 && (ld_out & 1) == 0 && (out_col & 1) == 0) {
        if (dtype == 1) return softmax_tc<__nv_bfloat16>(SA_TC_ARGS);
        return softmax_tc<__half>(SA_TC_ARGS);
    }
    long items = (long)B * S * heads;
    MIXERS_DISPATCH(dtype, softmax_attention_kernel<T><<<(unsigned)items, SA_WARPS * 32, smem, stream>>>(
        (const T*)q, q_ld, q_hs, (const T*)k, k_bs, k_ps, k_hs, (const T*)v, v_bs, v_ps, v_hs, B, S, heads, kv_heads, dim, vdim, held, shift, pad, window, chunk,
        scale, softcap, (const T*)sink, (T*)out, ld_out, out_col, dyn, rows16 ? 1 : 0));
    return mixers_status();
}

// floats of workspace that mixers_softmax_attention wants for these sizes (0: none; it then needs no workspace)
extern "C" long mixers_softmax_attention_workspace(int dtype, int B, int S, int heads, int kv_heads, int dim, int vdim) {
    if (B <= 0 || S <= 0 || !shared_head_ok(dtype, S, heads, kv_heads, dim, vdim)) return 0;
    const long tiles = (S * (heads / kv_heads) + 15) / 16;
    return (long)B * kv_heads * tiles * shared_head_splits(B, S, heads, kv_heads) * 16L * (vdim + 2);
}
