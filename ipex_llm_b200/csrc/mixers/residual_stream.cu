// The 32-bit residual stream of designs that normalise a sublayer's OUTPUT: token + bigram embedding, "x += norm(y) * scale"
// with the depth-weighted average of all earlier streams folded in, the RMS norm in front of the output head, and the
// element-wise activations between the matrix products (xIELU, silu(gate) * up, gelu(gate) * per-token table row).  All of
// them are bound by memory traffic: one pass over their rows, arithmetic in 32-bit floats.
#include "mixers_common.cuh"

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// block sum, the same value in every thread (added in warp order)
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();                                        // red may still be read from an earlier call
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float s = 0.0f;
    for (int i = 0; i < nw; ++i) s += red[i];
    return s;
}

// one block per token.  x = table[id] * scale (+ pair table row); a token's pair row is (previous id * mul_prev + id * mul_cur)
// mod buckets, row number `buckets` for a sequence's first token; the previous id of a call's first token comes from prev[b].
template <typename T>
__global__ void embed_pair_kernel(const T* __restrict__ table, float scale, const T* __restrict__ pair, long buckets, long mul_prev, long mul_cur,
                                  const int64_t* __restrict__ ids, const int64_t* __restrict__ prev, int B, int S, int width, int slot0,
                                  const int32_t* __restrict__ pad, float* __restrict__ x, float* __restrict__ x_copy, T* __restrict__ h) {
    const long n = blockIdx.x;
    const int b = (int)(n / S), t = (int)(n - (long)b * S);
    const int pos = slot0 + t - (pad ? pad[b] : 0);           // pad may be null: no new token is padding
    const long id = ids[n];
    long row = -1;
    if (pair && pos >= 0) {
        if (pos == 0) row = buckets;
        else {
            const long before = t > 0 ? ids[n - 1] : prev[b];
            row = (before * mul_prev + id * mul_cur) % buckets;
            if (row < 0) row += buckets;
        }
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = 0.0f;
        if (pos >= 0) {
            v = to_f(table[id * width + c]) * scale;
            if (row >= 0) v += to_f(pair[row * width + c]);
        }
        x[n * width + c] = v;
        if (x_copy) x_copy[n * width + c] = v;
        if (h) h[n * width + c] = from_f<T>(v);
    }
}

// one block per row:  x += y / rms(y) * gain * vec;  then, optionally, the new x is stored as stream number `index` of `stack`
// and replaced by sum_{j <= index} coef[j] * stack[j];  h = x in the model's type.
template <typename T, typename TY>
__global__ void rms_residual_kernel(float* __restrict__ x, const TY* __restrict__ y, const T* __restrict__ gain, const T* __restrict__ vec, float eps,
                                    int width, float* __restrict__ stack, long stack_stride, int index, const T* __restrict__ coef,
                                    T* __restrict__ h) {
    __shared__ float red[32];
    const long n = blockIdx.x;
    const TY* yr = y + n * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { float v = to_f(yr[c]); ss += v * v; }
    ss = block_sum(ss, red);
    float f = 1.0f / sqrtf(ss / (float)width + eps);
    if (gain) f *= to_f(gain[0]);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const long i = n * width + c;
        float u = to_f(yr[c]) * f;
        if (vec) u *= to_f(vec[c]);
        float v = x[i] + u;
        if (stack) {
            stack[index * stack_stride + i] = v;
            if (coef) {
                float a = 0.0f;
                for (int j = 0; j < index; ++j) a += to_f(coef[j]) * stack[j * stack_stride + i];
                v = a + to_f(coef[index]) * v;
            }
        }
        x[i] = v;
        if (h) h[i] = from_f<T>(v);
    }
}

// the same with a row's elements held in registers (rows up to 8 x blockDim wide): every global load -- y, x, the vector, the
// earlier streams of the depth average -- is issued before the row's sum is reduced, so a lone row (a decoding step) pays one
// round trip to memory instead of one per loop turn
constexpr int RR_MAXC = 8;
template <typename T, typename TY>
__global__ void rms_residual_cached_kernel(float* __restrict__ x, const TY* __restrict__ y, const T* __restrict__ gain, const T* __restrict__ vec,
                                           float eps, int width, float* __restrict__ stack, long stack_stride, int index,
                                           const T* __restrict__ coef, T* __restrict__ h) {
    __shared__ float red[32];
    const long base = (long)blockIdx.x * width;
    float yv[RR_MAXC], xv[RR_MAXC], vv[RR_MAXC], av[RR_MAXC];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < RR_MAXC; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        yv[k] = 0.0f; xv[k] = 0.0f; vv[k] = 1.0f; av[k] = 0.0f;
        if (c < width) {
            yv[k] = to_f(y[base + c]);
            xv[k] = x[base + c];
            if (vec) vv[k] = to_f(vec[c]);
        }
        ss += yv[k] * yv[k];
    }
    if (coef) {
        for (int j = 0; j < index; ++j) {
            const float cj = to_f(coef[j]);
            const float* sj = stack + j * stack_stride + base;
#pragma unroll
            for (int k = 0; k < RR_MAXC; ++k) {
                const int c = threadIdx.x + k * blockDim.x;
                if (c < width) av[k] += cj * sj[c];
            }
        }
    }
    ss = block_sum(ss, red);
    float f = 1.0f / sqrtf(ss / (float)width + eps);
    if (gain) f *= to_f(gain[0]);
    const float last = coef ? to_f(coef[index]) : 1.0f;
#pragma unroll
    for (int k = 0; k < RR_MAXC; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < width) {
            float v = xv[k] + yv[k] * f * vv[k];
            if (stack) {
                stack[index * stack_stride + base + c] = v;
                if (coef) v = av[k] + last * v;
            }
            x[base + c] = v;
            if (h) h[base + c] = from_f<T>(v);
        }
    }
}

// one block per row of a stream whose sublayers run side by side on two scalar-gain RMS norms of the same x:
//   x += y_a + y_c + y_b + y_d (each may be null; y_a, y_c in the model's type, y_b, y_d 32-bit);
//   pre_gain: x <- x / rms(x) * pre_gain[0] first (the norm behind an embedding);
//   stack: the new x is kept as stream `index`, and with coef replaced by sum_{j <= index} coef[j] * stack[j];
//   h1 = x / rms(x) * gain1[0], h2 = x / rms(x) * gain2[0] (either may be null): one root mean square serves both.
// CACHED: the row's elements stay in registers (rows up to SN_MAXC x blockDim wide), every load issued before the first reduction.
constexpr int SN_MAXC = 8;
template <typename T, bool CACHED>
__global__ void sum_residual_norms_kernel(float* __restrict__ x, int width, const T* __restrict__ y_a, const T* __restrict__ y_c,
                                          const float* __restrict__ y_b, const float* __restrict__ y_d, const T* __restrict__ pre_gain, float eps,
                                          float* __restrict__ stack, long stack_stride, int index, const T* __restrict__ coef,
                                          const T* __restrict__ gain1, const T* __restrict__ gain2, T* __restrict__ h1, T* __restrict__ h2) {
    __shared__ float red[32];
    const long base = (long)blockIdx.x * width;
    const bool want = h1 || h2;
    const float last = coef ? to_f(coef[index]) : 1.0f;
    auto summed = [&](long i) {
        float v = x[i];
        if (y_a) v += to_f(y_a[i]);
        if (y_c) v += to_f(y_c[i]);
        if (y_b) v += y_b[i];
        if (y_d) v += y_d[i];
        return v;
    };
    if (CACHED) {
        float v[SN_MAXC], av[SN_MAXC];
        float ss = 0.0f;
#pragma unroll
        for (int k = 0; k < SN_MAXC; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            v[k] = c < width ? summed(base + c) : 0.0f;
            av[k] = 0.0f;
            ss += v[k] * v[k];
        }
        if (coef) {
            for (int j = 0; j < index; ++j) {
                const float cj = to_f(coef[j]);
                const float* sj = stack + j * stack_stride + base;
#pragma unroll
                for (int k = 0; k < SN_MAXC; ++k) {
                    const int c = threadIdx.x + k * blockDim.x;
                    if (c < width) av[k] += cj * sj[c];
                }
            }
        }
        if (pre_gain) {
            const float f = to_f(pre_gain[0]) / sqrtf(block_sum(ss, red) / (float)width + eps);
#pragma unroll
            for (int k = 0; k < SN_MAXC; ++k) v[k] *= f;
        }
        ss = 0.0f;
#pragma unroll
        for (int k = 0; k < SN_MAXC; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < width) {
                if (stack) {
                    stack[index * stack_stride + base + c] = v[k];
                    if (coef) v[k] = av[k] + last * v[k];
                }
                x[base + c] = v[k];
            }
            ss += v[k] * v[k];
        }
        if (!want) return;
        const float f = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
        const float f1 = h1 ? f * to_f(gain1[0]) : 0.0f, f2 = h2 ? f * to_f(gain2[0]) : 0.0f;
#pragma unroll
        for (int k = 0; k < SN_MAXC; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < width) {
                if (h1) h1[base + c] = from_f<T>(v[k] * f1);
                if (h2) h2[base + c] = from_f<T>(v[k] * f2);
            }
        }
        return;
    }
    // every thread re-reads only what it wrote itself
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = summed(base + c); x[base + c] = v; ss += v * v; }
    const float f0 = pre_gain ? to_f(pre_gain[0]) / sqrtf(block_sum(ss, red) / (float)width + eps) : 1.0f;
    if (pre_gain || stack) {
        ss = 0.0f;
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            const long i = base + c;
            float v = x[i] * f0;
            if (stack) {
                stack[index * stack_stride + i] = v;
                if (coef) {
                    float a = 0.0f;
                    for (int j = 0; j < index; ++j) a += to_f(coef[j]) * stack[j * stack_stride + i];
                    v = a + last * v;
                }
            }
            x[i] = v;
            ss += v * v;
        }
    }
    if (!want) return;
    const float f = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    const float f1 = h1 ? f * to_f(gain1[0]) : 0.0f, f2 = h2 ? f * to_f(gain2[0]) : 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = x[base + c];
        if (h1) h1[base + c] = from_f<T>(v * f1);
        if (h2) h2[base + c] = from_f<T>(v * f2);
    }
}

// out[n, c] = gelu(in[n, c]) with the exact (erf) form
template <typename T>
__global__ void gelu_erf_kernel(const T* __restrict__ in, long n, T* __restrict__ out) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float v = to_f(in[i]);
        out[i] = from_f<T>(0.5f * v * (1.0f + erff(v * 0.7071067811865476f)));
    }
}

// one block per row: out = x / rms(x) * gain * vec
template <typename T>
__global__ void rms_norm_rows_kernel(const float* __restrict__ x, const T* __restrict__ gain, const T* __restrict__ vec, float eps, int width,
                                     T* __restrict__ out) {
    __shared__ float red[32];
    const long n = blockIdx.x;
    const float* xr = x + n * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { float v = xr[c]; ss += v * v; }
    ss = block_sum(ss, red);
    float f = 1.0f / sqrtf(ss / (float)width + eps);
    if (gain) f *= to_f(gain[0]);
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[n * width + c] = from_f<T>(xr[c] * f * (vec ? to_f(vec[c]) : 1.0f));
}

// xIELU, with a = softplus(p) and c = 1/2 + softplus(q): f(z) = a z^2 + z/2 where z is positive, c (expm1(z) - z) + z/2 elsewhere
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ z, long n, const T* __restrict__ pq, T* __restrict__ out) {
    const float ap = softplus_f(to_f(pq[0])), aq = 0.5f + softplus_f(to_f(pq[1]));
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const float v = to_f(z[i]);
        out[i] = from_f<T>(v > 0.0f ? ap * v * v + 0.5f * v : aq * (expm1f(v) - v) + 0.5f * v);
    }
}

// out[n, c] = silu(in[n, off_gate + c]) * in[n, off_up + c]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, long n_rows, int ld, int off_gate, int off_up, int cols, T* __restrict__ out) {
    const long total = n_rows * cols;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long n = i / cols;
        const int c = (int)(i - n * cols);
        const T* r = in + n * ld;
        out[i] = from_f<T>(silu_f(to_f(r[off_gate + c])) * to_f(r[off_up + c]));
    }
}

// out[n, c] = g' sigmoid(1.702 g') (u' + 1), g' = min(in[n, off_gate + c], limit), u' = clamp(in[n, off_up + c], -limit, limit)
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ in, long n_rows, int ld, int off_gate, int off_up, int cols, float limit, T* __restrict__ out) {
    const long total = n_rows * cols;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long n = i / cols;
        const int c = (int)(i - n * cols);
        const float g = fminf(to_f(in[n * ld + off_gate + c]), limit);
        const float u = fminf(fmaxf(to_f(in[n * ld + off_up + c]), -limit), limit);
        out[i] = from_f<T>(g * sigmoid_f(1.702f * g) * (u + 1.0f));
    }
}

// out[n, c] = gelu_tanh(g[n, c]) * table[ids[n], col0 + c]
template <typename T>
__global__ void gelu_table_mul_kernel(const T* __restrict__ g, long n_rows, int cols, const T* __restrict__ table, int ld_table, int col0,
                                      const int64_t* __restrict__ ids, T* __restrict__ out) {
    const long total = n_rows * cols;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long n = i / cols;
        const int c = (int)(i - n * cols);
        out[i] = from_f<T>(gelu_tanh_f(to_f(g[i])) * to_f(table[ids[n] * ld_table + col0 + c]));
    }
}

static inline int grid_for(long n) {
    long b = (n + 255) / 256;
    return (int)(b < 1 ? 1 : (b > 148L * 16 ? 148L * 16 : b));
}

extern "C" int mixers_embed_pair(int dtype, const void* table, float scale, const void* pair, long buckets, long mul_prev, long mul_cur,
                                 const int64_t* ids, const int64_t* prev, int B, int S, int width, int slot0, const int32_t* pad, float* x,
                                 float* x_copy, void* h, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (pair && buckets < 1) return (int)cudaErrorInvalidValue;
    const int threads = width >= 256 ? 256 : 128;
    MIXERS_DISPATCH(dtype, embed_pair_kernel<T><<<(unsigned)((long)B * S), threads, 0, (cudaStream_t)stream>>>(
        (const T*)table, scale, (const T*)pair, buckets, mul_prev, mul_cur, ids, prev, B, S, width, slot0, pad, x, x_copy, (T*)h));
    return mixers_status();
}

extern "C" int mixers_rms_residual(int dtype, float* x, long n_rows, int width, const void* y, int y_is_float, const void* gain, const void* vec,
                                   float eps, float* stack, long stack_stride, int index, const void* coef, void* h, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    if (coef && !stack) return (int)cudaErrorInvalidValue;
    // many rows keep the memory system busy by themselves, and the depth average then streams better from the plain loop
    if (width <= RR_MAXC * 1024 && (n_rows <= 1024 || !coef)) {
        int cached = ((width + RR_MAXC - 1) / RR_MAXC + 31) / 32 * 32;
        if (cached < 64) cached = 64;
        if (y_is_float) {
            MIXERS_DISPATCH(dtype, rms_residual_cached_kernel<T, float><<<(unsigned)n_rows, cached, 0, (cudaStream_t)stream>>>(
                x, (const float*)y, (const T*)gain, (const T*)vec, eps, width, stack, stack_stride, index, (const T*)coef, (T*)h));
        } else {
            MIXERS_DISPATCH(dtype, rms_residual_cached_kernel<T, T><<<(unsigned)n_rows, cached, 0, (cudaStream_t)stream>>>(
                x, (const T*)y, (const T*)gain, (const T*)vec, eps, width, stack, stack_stride, index, (const T*)coef, (T*)h));
        }
        return mixers_status();
    }
    const int threads = width >= 1024 ? 256 : 128;
    if (y_is_float) {
        MIXERS_DISPATCH(dtype, rms_residual_kernel<T, float><<<(unsigned)n_rows, threads, 0, (cudaStream_t)stream>>>(
            x, (const float*)y, (const T*)gain, (const T*)vec, eps, width, stack, stack_stride, index, (const T*)coef, (T*)h));
    } else {
        MIXERS_DISPATCH(dtype, rms_residual_kernel<T, T><<<(unsigned)n_rows, threads, 0, (cudaStream_t)stream>>>(
            x, (const T*)y, (const T*)gain, (const T*)vec, eps, width, stack, stack_stride, index, (const T*)coef, (T*)h));
    }
    return mixers_status();
}

extern "C" int mixers_rms_norm_rows(int dtype, const float* x, long n_rows, int width, const void* gain, const void* vec, float eps, void* out,
                                    mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    MIXERS_DISPATCH(dtype, rms_norm_rows_kernel<T><<<(unsigned)n_rows, threads, 0, (cudaStream_t)stream>>>(
        x, (const T*)gain, (const T*)vec, eps, width, (T*)out));
    return mixers_status();
}

extern "C" int mixers_xielu(int dtype, const void* z, long n, const void* pq, void* out, mixers_stream_t stream) {
    if (n <= 0) return 0;
    MIXERS_DISPATCH(dtype, xielu_kernel<T><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const T*)z, n, (const T*)pq, (T*)out));
    return mixers_status();
}

extern "C" int mixers_silu_mul(int dtype, const void* in, long n_rows, int ld, int off_gate, int off_up, int cols, void* out,
                               mixers_stream_t stream) {
    if (n_rows <= 0 || cols <= 0) return 0;
    MIXERS_DISPATCH(dtype, silu_mul_kernel<T><<<grid_for(n_rows * cols), 256, 0, (cudaStream_t)stream>>>(
        (const T*)in, n_rows, ld, off_gate, off_up, cols, (T*)out));
    return mixers_status();
}

extern "C" int mixers_gelu_table_mul(int dtype, const void* g, long n_rows, int cols, const void* table, int ld_table, int col0,
                                     const int64_t* ids, void* out, mixers_stream_t stream) {
    if (n_rows <= 0 || cols <= 0) return 0;
    MIXERS_DISPATCH(dtype, gelu_table_mul_kernel<T><<<grid_for(n_rows * cols), 256, 0, (cudaStream_t)stream>>>(
        (const T*)g, n_rows, cols, (const T*)table, ld_table, col0, ids, (T*)out));
    return mixers_status();
}

extern "C" int mixers_clamped_glu(int dtype, const void* in, long n_rows, int ld, int off_gate, int off_up, int cols, float limit, void* out,
                                  mixers_stream_t stream) {
    if (n_rows <= 0 || cols <= 0) return 0;
    MIXERS_DISPATCH(dtype, clamped_glu_kernel<T><<<grid_for(n_rows * cols), 256, 0, (cudaStream_t)stream>>>((const T*)in, n_rows, ld, off_gate, off_up, cols,
                                                                                                          limit, (T*)out));
    return mixers_status();
}

extern "C" int mixers_sum_residual_norms(int dtype, float* x, long n_rows, int width, const void* y_a, const void* y_c, const float* y_b,
                                         const float* y_d, const void* pre_gain, float eps, float* stack, long stack_stride, int index,
                                         const void* coef, const void* gain1, const void* gain2, void* h1, void* h2, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    if ((coef && !stack) || (h1 && !gain1) || (h2 && !gain2)) return (int)cudaErrorInvalidValue;
    int threads = width > 1024 ? 256 : 128;
    if (n_rows <= 64)                                        // a decoding step's few rows: one round trip to memory for rows up to 8192 wide
        while (threads < 1024 && threads * SN_MAXC < width) threads <<= 1;
    // many rows under a depth average stream better from the plain loop
    const bool cached = width <= SN_MAXC * threads && (n_rows <= 1024 || !coef);
#define SN_LAUNCH(C) MIXERS_DISPATCH(dtype, sum_residual_norms_kernel<T, C><<<(unsigned)n_rows, threads, 0, (cudaStream_t)stream>>>(                    \
        x, width, (const T*)y_a, (const T*)y_c, y_b, y_d, (const T*)pre_gain, eps, stack, stack_stride, index, (const T*)coef, (const T*)gain1, \
        (const T*)gain2, (T*)h1, (T*)h2))
    if (cached) SN_LAUNCH(true);
    else SN_LAUNCH(false);
#undef SN_LAUNCH
    return mixers_status();
}

extern "C" int mixers_gelu_erf(int dtype, const void* in, long n, void* out, mixers_stream_t stream) {
    if (n <= 0) return 0;
    MIXERS_DISPATCH(dtype, gelu_erf_kernel<T><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const T*)in, n, (T*)out));
    return mixers_status();
}
