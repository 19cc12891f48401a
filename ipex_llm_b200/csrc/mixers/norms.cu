// Normalisations and other row-wise pieces: embedding gather into the 32-bit residual stream, Dynamic Tanh fused with the
// residual update, layer norm (weight only) fused with the residual update of a layer whose sublayers run side by side, gated RMS output norm of the recurrences, PolyNorm, soft-capped logits.  All of them are bound by memory
// traffic: one pass over their rows, arithmetic in 32-bit floats.
#include "mixers_common.cuh"

template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids, long n_rows, int width, float* __restrict__ x) {
    long total = n_rows * (long)width;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        long n = i / width;
        int c = (int)(i - n * width);
        x[i] = to_f(table[ids[n] * (long)width + c]);
    }
}

// one block row per token (blockIdx.x), columns across the block and blockIdx.y
template <typename T>
__global__ void dyt_residual_norm_kernel(float* __restrict__ x, long n_rows, int width, const T* __restrict__ y, const T* __restrict__ post_w,
                                         const T* __restrict__ post_b, const T* __restrict__ post_alpha, const T* __restrict__ add,
                                         const T* __restrict__ pre_w, const T* __restrict__ pre_b, const T* __restrict__ pre_alpha,
                                         T* __restrict__ out) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const long i = (long)blockIdx.x * width + c;
    float v = x[i];
    if (y) v += tanhf(to_f(post_alpha[0]) * to_f(y[i])) * to_f(post_w[c]) + to_f(post_b[c]);
    if (add) v += to_f(add[c]);
    if (y || add) x[i] = v;
    if (out) out[i] = from_f<T>(tanhf(to_f(pre_alpha[0]) * v) * to_f(pre_w[c]) + to_f(pre_b[c]));
}

// one block per row: x += (y_a + y_b) (either may be null; y_a in the model's type, y_b 32-bit), then out = layer norm of the new
// x (mean removed, over the standard deviation, times w; no bias).  A row that fits LN_MAXC elements a thread is held in
// registers (one round trip to memory), a wider one is read three times.  A prompt's many rows run in blocks of 128 threads
// (many blocks per SM; the re-reads come from the caches); the few rows of a decoding step, which pay latency and nothing else,
// get blocks of up to 1024 threads so that rows up to 8192 wide stay in registers.
constexpr int LN_MAXC = 8, LN_FEW_ROWS = 64;
template <int LN_THREADS>
__device__ __forceinline__ float ln_block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < LN_THREADS / 32; ++i) s += red[i];
    return s;
}

template <typename T, int LN_THREADS>
__global__ void __launch_bounds__(LN_THREADS) layer_norm_residual_kernel(float* __restrict__ x, int width, const T* __restrict__ y_a,
                                                                       const float* __restrict__ y_b, const T* __restrict__ w, float eps,
                                                                       T* __restrict__ out) {
    __shared__ float red[LN_THREADS / 32];
    const long base = (long)blockIdx.x * width;
    const bool add = y_a || y_b;
    if (width <= LN_MAXC * LN_THREADS) {
        float v[LN_MAXC];
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < LN_MAXC; ++k) {
            const int c = threadIdx.x + k * LN_THREADS;
            v[k] = 0.0f;
            if (c < width) {
                float a = y_a ? to_f(y_a[base + c]) : 0.0f;
                if (y_b) a += y_b[base + c];
                v[k] = add ? x[base + c] + a : x[base + c];
                if (add) x[base + c] = v[k];
                sum += v[k];
            }
        }
        if (!out) return;
        const float mean = ln_block_sum<LN_THREADS>(sum, red) / (float)width;
        float sq = 0.0f;
#pragma unroll
        for (int k = 0; k < LN_MAXC; ++k) {
            const int c = threadIdx.x + k * LN_THREADS;
            if (c < width) { v[k] -= mean; sq += v[k] * v[k]; }
        }
        const float inv = 1.0f / sqrtf(ln_block_sum<LN_THREADS>(sq, red) / (float)width + eps);
#pragma unroll
        for (int k = 0; k < LN_MAXC; ++k) {
            const int c = threadIdx.x + k * LN_THREADS;
            if (c < width) out[base + c] = from_f<T>(v[k] * inv * to_f(w[c]));
        }
        return;
    }
    float sum = 0.0f;
    for (int c = threadIdx.x; c < width; c += LN_THREADS) {
        float v = x[base + c];
        if (add) {
            float a = y_a ? to_f(y_a[base + c]) : 0.0f;
            if (y_b) a += y_b[base + c];
            v += a;
            x[base + c] = v;
        }
        sum += v;
    }
    if (!out) return;
    const float mean = ln_block_sum<LN_THREADS>(sum, red) / (float)width;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < width; c += LN_THREADS) { const float d = x[base + c] - mean; sq += d * d; }
    const float inv = 1.0f / sqrtf(ln_block_sum<LN_THREADS>(sq, red) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += LN_THREADS) out[base + c] = from_f<T>((x[base + c] - mean) * inv * to_f(w[c]));
}

// one warp per (row, head); w_head_stride: 0 = one weight vector [vdim] for every head, vdim = a vector per head [heads * vdim].
// gate_mode bit 0: the gate is sigmoid(g) instead of silu(g); bit 1: the gate multiplies BEFORE the norm (the root mean square is
// that of the gated values) instead of after it
template <typename T>
__global__ void gated_rms_norm_kernel(const float* __restrict__ o, long n_rows, int heads, int vdim, const T* __restrict__ gate, int ld_gate,
                                      int off_g, const T* __restrict__ w, int w_head_stride, float eps, T* __restrict__ out, int ld_out, int out_col,
                                      float out_scale, int gate_mode) {
    long warp = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= n_rows * heads) return;
    long n = warp / heads;
    int h = (int)(warp - n * heads);
    const float* src = o + warp * (long)vdim;
    const T* g = gate + n * (long)ld_gate + off_g + h * vdim;
    auto gated = [&](int c) { const float z = to_f(g[c]); return (gate_mode & 1) ? sigmoid_f(z) : silu_f(z); };
    const bool first = (gate_mode & 2) != 0;
    float ss = 0.0f;
    for (int c = lane; c < vdim; c += 32) { float v = first ? src[c] * gated(c) : src[c]; ss += v * v; }
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    T* dst = out + n * (long)ld_out + out_col + h * vdim;
    w += (long)h * w_head_stride;
    for (int c = lane; c < vdim; c += 32)
        dst[c] = from_f<T>(src[c] * inv * to_f(w[c]) * gated(c) * out_scale);
}

// the same for wide heads (a state-space branch normalises its whole inner width in a few parts): one block per (row, head), the
// head's values -- gated already when the gate comes first -- stay in registers between the sum of squares and the write
constexpr int GN_MAXC = 8;
__device__ __forceinline__ float gn_block_sum(float v, float* red) {
    v = warp_sum(v);
    const int nw = (blockDim.x + 31) >> 5;
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
    for (int i = 0; i < nw; ++i) s += red[i];
    return s;
}

template <typename T>
__global__ void gated_rms_norm_wide_kernel(const float* __restrict__ o, int heads, int vdim, const T* __restrict__ gate, int ld_gate, int off_g,
                                           const T* __restrict__ w, int w_head_stride, float eps, T* __restrict__ out, int ld_out, int out_col,
                                           float out_scale, int gate_mode) {
    __shared__ float red[32];
    const long item = blockIdx.x;
    const long n = item / heads;
    const int h = (int)(item - n * heads);
    const float* src = o + item * (long)vdim;
    const T* g = gate + n * (long)ld_gate + off_g + h * vdim;
    const bool first = (gate_mode & 2) != 0;
    float v[GN_MAXC], gt[GN_MAXC];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < GN_MAXC; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = 0.0f; gt[k] = 0.0f;
        if (c < vdim) {
            const float z = to_f(g[c]);
            gt[k] = (gate_mode & 1) ? sigmoid_f(z) : silu_f(z);
            v[k] = first ? src[c] * gt[k] : src[c];
            ss += v[k] * v[k];
        }
    }
    const float inv = out_scale / sqrtf(gn_block_sum(ss, red) / (float)vdim + eps);
    T* dst = out + n * (long)ld_out + out_col + h * vdim;
    w += (long)h * w_head_stride;
#pragma unroll
    for (int k = 0; k < GN_MAXC; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < vdim) dst[c] = from_f<T>(v[k] * inv * to_f(w[c]) * (first ? 1.0f : gt[k]));
    }
}

// o[n, c] *= sigmoid(gate[n, off_g + c / per_gate]) in place: a gate per channel (per_gate 1) or one per head (per_gate = the
// head's channels)
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, long n_rows, int cols, const T* __restrict__ gate, int ld_gate, int off_g, int per_gate) {
    const long total = n_rows * cols;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long n = i / cols;
        const int c = (int)(i - n * cols);
        o[i] = from_f<T>(to_f(o[i]) * sigmoid_f(to_f(gate[n * ld_gate + off_g + c / per_gate])));
    }
}

// one block per row: out = scale * (a / rms(a) * w_a + b / rms(b) * w_b), 32-bit out (two branch outputs meet as normalised vectors)
template <typename T>
__global__ void rms_pair_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ w_a, const T* __restrict__ w_b, float eps,
                                    float scale, int width, float* __restrict__ out) {
    __shared__ float red[2][32];
    const long base = (long)blockIdx.x * width;
    float sa = 0.0f, sb = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float u = to_f(a[base + c]), v = to_f(b[base + c]); sa += u * u; sb += v * v; }
    sa = warp_sum(sa); sb = warp_sum(sb);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) { red[0][wid] = sa; red[1][wid] = sb; }
    __syncthreads();
    sa = sb = 0.0f;
    for (int i = 0; i < nw; ++i) { sa += red[0][i]; sb += red[1][i]; }
    const float fa = scale / sqrtf(sa / (float)width + eps), fb = scale / sqrtf(sb / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[base + c] = to_f(a[base + c]) * fa * to_f(w_a[c]) + to_f(b[base + c]) * fb * to_f(w_b[c]);
}

// one block per row
template <typename T>
__global__ void poly_norm_kernel(const T* __restrict__ z, long n_rows, int width, const T* __restrict__ coef, float eps, T* __restrict__ out) {
    __shared__ float red[3][32];
    long n = blockIdx.x;
    const T* src = z + n * (long)width;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = to_f(src[c]);
        float v2 = v * v;
        s2 += v2; s4 += v2 * v2; s6 += v2 * v2 * v2;
    }
    s2 = warp_sum(s2); s4 = warp_sum(s4); s6 = warp_sum(s6);
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { red[0][wid] = s2; red[1][wid] = s4; red[2][wid] = s6; }
    __syncthreads();
    s2 = s4 = s6 = 0.0f;
    for (int i = 0; i < nw; ++i) { s2 += red[0][i]; s4 += red[1][i]; s6 += red[2][i]; }      // same order in every thread
    float r1 = 1.0f / sqrtf(s2 / (float)width + eps), r2 = 1.0f / sqrtf(s4 / (float)width + eps), r3 = 1.0f / sqrtf(s6 / (float)width + eps);
    float a = to_f(coef[0]) * r1, b = to_f(coef[1]) * r2, cc = to_f(coef[2]) * r3, e = to_f(coef[3]);
    T* dst = out + n * (long)width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = to_f(src[c]);
        dst[c] = from_f<T>(a * v + b * (v * v) + cc * (v * v * v) + e);
    }
}

template <typename T>
__global__ void soft_cap_kernel(const T* __restrict__ x, long n, float cap, float* __restrict__ out) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        float v = to_f(x[i]);
        out[i] = cap > 0.0f ? cap * tanhf(v / cap) : v;
    }
}

static inline int grid_for(long total, int block) {
    long g = (total + block - 1) / block;
    return (int)(g < 1 ? 1 : (g > 148L * 32 ? 148L * 32 : g));
}

extern "C" int mixers_embed_rows(int dtype, const void* table, const int64_t* ids, long n_rows, int width, float* x, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    MIXERS_DISPATCH(dtype, embed_rows_kernel<T><<<grid_for(n_rows * width, 256), 256, 0, (cudaStream_t)stream>>>((const T*)table, ids, n_rows, width, x));
    return mixers_status();
}

extern "C" int mixers_dyt_residual_norm(int dtype, float* x, long n_rows, int width, const void* y, const void* post_w, const void* post_b,
                                        const void* post_alpha, const void* add, const void* pre_w, const void* pre_b, const void* pre_alpha,
                                        void* out, mixers_stream_t stream) {
    if (n_rows <= 0 || (!y && !add && !out)) return 0;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    dim3 blocks((unsigned)n_rows, (unsigned)((width + threads - 1) / threads));
    MIXERS_DISPATCH(dtype, dyt_residual_norm_kernel<T><<<blocks, threads, 0, (cudaStream_t)stream>>>(
        x, n_rows, width, (const T*)y, (const T*)post_w, (const T*)post_b, (const T*)post_alpha, (const T*)add, (const T*)pre_w,
        (const T*)pre_b, (const T*)pre_alpha, (T*)out));
    return mixers_status();
}

extern "C" int mixers_layer_norm_residual(int dtype, float* x, long n_rows, int width, const void* y_a, const float* y_b, const void* w, float eps,
                                          void* out, mixers_stream_t stream) {
    if (n_rows <= 0 || (!y_a && !y_b && !out)) return 0;
    if (out && !w) return (int)cudaErrorInvalidValue;
    int threads = 128;
    if (n_rows <= LN_FEW_ROWS)
        while (threads < 1024 && threads * LN_MAXC < width) threads <<= 1;
#define LN_LAUNCH(TH) MIXERS_DISPATCH(dtype, layer_norm_residual_kernel<T, TH><<<(unsigned)n_rows, TH, 0, (cudaStream_t)stream>>>( \
        x, width, (const T*)y_a, y_b, (const T*)w, eps, (T*)out))
    if (threads == 128) LN_LAUNCH(128);
    else if (threads == 256) LN_LAUNCH(256);
    else if (threads == 512) LN_LAUNCH(512);
    else LN_LAUNCH(1024);
#undef LN_LAUNCH
    return mixers_status();
}

extern "C" int mixers_gated_rms_norm(int dtype, const float* o, long n_rows, int heads, int vdim, const void* gate, int ld_gate, int off_g,
                                     const void* w, int w_head_stride, float eps, void* out, int ld_out, int out_col, float out_scale,
                                     int gate_mode, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    if (gate_mode & ~3) return (int)cudaErrorInvalidValue;
    long warps = n_rows * heads;
    if (vdim > 256 && vdim <= GN_MAXC * 1024 && warps <= 1024) {   // few wide heads (a decoding step): a block each; many rows keep every SM
                                                                    // busy with a warp each
        int threads = 128;
        while (threads < 1024 && threads * GN_MAXC < vdim) threads <<= 1;
        if (threads * 4 <= vdim && threads < 1024) threads <<= 1;   // at least two rounds of loads in flight per thread are enough
        MIXERS_DISPATCH(dtype, gated_rms_norm_wide_kernel<T><<<(unsigned)warps, threads, 0, (cudaStream_t)stream>>>(
            o, heads, vdim, (const T*)gate, ld_gate, off_g, (const T*)w, w_head_stride, eps, (T*)out, ld_out, out_col, out_scale, gate_mode));
        return mixers_status();
    }
    int blocks = (int)((warps + 3) / 4);
    MIXERS_DISPATCH(dtype, gated_rms_norm_kernel<T><<<blocks, 128, 0, (cudaStream_t)stream>>>(o, n_rows, heads, vdim, (const T*)gate, ld_gate, off_g,
                                                                                                (const T*)w, w_head_stride, eps, (T*)out, ld_out, out_col,
                                                                                                out_scale, gate_mode));
    return mixers_status();
}

extern "C" int mixers_poly_norm(int dtype, const void* z, long n_rows, int width, const void* coef, float eps, void* out, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    MIXERS_DISPATCH(dtype, poly_norm_kernel<T><<<(int)n_rows, 256, 0, (cudaStream_t)stream>>>((const T*)z, n_rows, width, (const T*)coef, eps, (T*)out));
    return mixers_status();
}

extern "C" int mixers_soft_cap(int dtype, const void* x, long n, float cap, float* out, mixers_stream_t stream) {
    if (n <= 0) return 0;
    MIXERS_DISPATCH(dtype, soft_cap_kernel<T><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const T*)x, n, cap, out));
    return mixers_status();
}

extern "C" int mixers_sigmoid_gate(int dtype, void* o, long n_rows, int cols, const void* gate, int ld_gate, int off_g, int per_gate,
                                   mixers_stream_t stream) {
    if (n_rows <= 0 || cols <= 0) return 0;
    if (per_gate < 1) return (int)cudaErrorInvalidValue;
    MIXERS_DISPATCH(dtype, sigmoid_gate_kernel<T><<<grid_for(n_rows * cols, 256), 256, 0, (cudaStream_t)stream>>>((T*)o, n_rows, cols, (const T*)gate,
                                                                                                                 ld_gate, off_g, per_gate));
    return mixers_status();
}

extern "C" int mixers_rms_pair_sum(int dtype, const void* a, const void* b, const void* w_a, const void* w_b, float eps, float scale, long n_rows,
                                   int width, float* out, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    MIXERS_DISPATCH(dtype, rms_pair_sum_kernel<T><<<(unsigned)n_rows, threads, 0, (cudaStream_t)stream>>>((const T*)a, (const T*)b, (const T*)w_a,
                                                                                                        (const T*)w_b, eps, scale, width, out));
    return mixers_status();
}
