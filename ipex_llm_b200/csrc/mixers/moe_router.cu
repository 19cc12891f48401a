// Mixture-of-experts routing with groups and identity experts, and the pieces around the experts' matrix products:
//   scored_router: 32-bit router logits, scores = softmax over all outputs or a sigmoid each, a correction that enters the
//     ranking but not the weights, consecutive outputs ranked as groups first (by the sum of their best few members; only the
//     leading groups stay eligible), then top-k among the eligible; weights = the winners' scores, optionally divided by
//     their sum and scaled; one more row of the same product may gate a shared expert (sigmoid of its logit);
//   gated activations of an expert: silu(g) u, or the clamped form g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit),
//     u' = clamp(u, -limit, limit);
//   moe_small_up / moe_small_down: the chosen experts of a few tokens straight from the experts' weight matrices (device
//     tables of addresses), nothing on the host between router and result: the path of decoding and of a recorded step;
//   moe_sort / moe_combine: many tokens -- the (token, choice) pairs counted and sorted by expert on the device, then the
//     weighted sum of the expert outputs that were computed expert by expert on the sorted rows.
// Outputs numbered >= n_experts are identity experts: their output is the token's input itself.
#include "mixers_common.cuh"
#include <math.h>

constexpr int ROUTER_WARPS = 32, ROUTER_WARPS_MANY = 8, ROUTER_FEW_ROWS = 64;

// lowest index among the largest values of vals[0..n) that are still allowed (taken[i] == 0); one warp
__device__ __forceinline__ int warp_argmax(const float* vals, const unsigned char* blocked, int n, int lane) {
    float best = -INFINITY;
    int at = -1;
    for (int i = lane; i < n; i += 32) {
        if (blocked[i]) continue;
        const float v = vals[i];
        if (at < 0 || v > best) { best = v; at = i; }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, m);
        const int oa = __shfl_xor_sync(0xffffffffu, at, m);
        if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
    }
    return at;
}

template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ a, const T* __restrict__ b, int n, int lane) {
    float s = 0.0f;
    if constexpr (sizeof(T) == 2) {
        if ((n & 7) == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
            for (int c = lane * 8; c < n; c += 256) {
                uint4 va = *reinterpret_cast<const uint4*>(a + c), vb = *reinterpret_cast<const uint4*>(b + c);
                const T* ea = reinterpret_cast<const T*>(&va);
                const T* eb = reinterpret_cast<const T*>(&vb);
#pragma unroll
                for (int i = 0; i < 8; ++i) s += to_f(ea[i]) * to_f(eb[i]);
            }
            return warp_sum(s);
        }
    }
    for (int c = lane; c < n; c += 32) s += to_f(a[c]) * to_f(b[c]);
    return warp_sum(s);
}

// a . (b * w) with the scaled b rounded to the model's type first (an expert that is fed its weighted input)
template <typename T>
__device__ __forceinline__ float warp_dot_scaled(const T* __restrict__ a, const T* __restrict__ b, int n, int lane, float w) {
    float s = 0.0f;
    for (int c = lane; c < n; c += 32) s += to_f(a[c]) * to_f(from_f<T>(to_f(b[c]) * w));
    return warp_sum(s);
}

// one block of ROUTER_WARPS warps per token.  The rows of the product (the router's and, if given, the shared expert's gate row)
// are cut into `split` pieces each and the pieces dealt to the warps (16-byte loads): a decoding step's lone token pays the
// latency of one short piece, not of whole rows one after another.  Few tokens get blocks of ROUTER_WARPS warps, a prompt's many
// tokens blocks of ROUTER_WARPS_MANY (more blocks per SM); the cut and the order in which the pieces are added are the same in
// both, so a token's logits do not depend on the batch.  Warp 0 then chooses.
template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32) scored_router_kernel(
        const T* __restrict__ h, long n_rows, int width, const T* __restrict__ router, const T* __restrict__ correction, int n_out, int groups,
        int keep, int top, int score_mode, int group_top, int renorm, float w_scale, const T* __restrict__ gate_row, float* __restrict__ gate_out,
        int split, int32_t* __restrict__ idx_out, float* __restrict__ w_out) {
    extern __shared__ float router_sh[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = n_out + (gate_row ? 1 : 0);
    float* part = router_sh;                                // [rows * split] partial products
    float* score = part + rows * split;                     // logits, then scores
    float* choice = score + n_out;                          // scores + correction
    float* gbest = choice + n_out;
    unsigned char* blocked = reinterpret_cast<unsigned char*>(gbest + groups);      // [n_out] experts, then [groups]
    unsigned char* gblocked = blocked + n_out;
    const long n = blockIdx.x;
    const T* hr = h + n * width;
    const int chunk = ((width + split - 1) / split + 7) & ~7;                  // a multiple of 8: pieces keep the rows' alignment
    for (int item = wid; item < rows * split; item += (int)(blockDim.x >> 5)) {
        const int e = item / split, c0 = (item - e * split) * chunk;
        const int len = width - c0 < chunk ? width - c0 : chunk;
        const T* wr = e < n_out ? router + (long)e * width : gate_row;           // row n_out: the shared expert's gate
        const float s = len > 0 ? warp_dot(wr + c0, hr + c0, len, lane) : 0.0f;
        if (lane == 0) part[item] = s;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < rows; e += blockDim.x) {
        float s = 0.0f;
        for (int i = 0; i < split; ++i) s += part[e * split + i];
        if (e < n_out) score[e] = s;
        else gate_out[n] = sigmoid_f(s);
    }
    __syncthreads();
    if (wid != 0) return;
    float big = -INFINITY, sum = 1.0f;
    if (score_mode == 0) {
        for (int e = lane; e < n_out; e += 32) big = fmaxf(big, score[e]);
        big = warp_max(big);
        sum = 0.0f;
        for (int e = lane; e < n_out; e += 32) sum += expf(score[e] - big);
        sum = warp_sum(sum);
    }
    for (int e = lane; e < n_out; e += 32) {
        const float s = score_mode == 0 ? expf(score[e] - big) / sum : sigmoid_f(score[e]);
        score[e] = s;
        choice[e] = correction ? s + to_f(correction[e]) : s;
        blocked[e] = 1;
    }
    __syncwarp();
    const int per = n_out / groups;
    for (int g = lane; g < groups; g += 32) {
        // the sum of the group's group_top largest choice scores (all of them if it has fewer members)
        float b = 0.0f, last = INFINITY;
        int last_i = -1;
        for (int r = 0; r < group_top && r < per; ++r) {    // next largest: below the last taken, or equal with a higher index
            float best = -INFINITY;
            int at = -1;
            for (int i = 0; i < per; ++i) {
                const float v = choice[g * per + i];
                const bool after = v < last || (v == last && i > last_i);
                if (after && (at < 0 || v > best)) { best = v; at = i; }
            }
            if (at < 0) break;
            b += best; last = best; last_i = at;
        }
        gbest[g] = b;
        gblocked[g] = 0;
    }
    __syncwarp();
    for (int r = 0; r < keep; ++r) {                        // the best groups: their members may be chosen
        const int g = warp_argmax(gbest, gblocked, groups, lane);
        if (g < 0) break;
        if (lane == 0) gblocked[g] = 1;
        for (int i = lane; i < per; i += 32) blocked[g * per + i] = 0;
        __syncwarp();
    }
    float chosen_sum = 0.0f;
    for (int r = 0; r < top; ++r) {
        const int e = warp_argmax(choice, blocked, n_out, lane);
        if (lane == 0) {
            idx_out[n * top + r] = e < 0 ? n_out : e;       // n_out: nothing left to choose (weight 0)
            w_out[n * top + r] = e < 0 ? 0.0f : score[e];
            if (e >= 0) { blocked[e] = 1; chosen_sum += score[e]; }
        }
        __syncwarp();
    }
    if (lane == 0 && (renorm || w_scale != 1.0f)) {
        const float f = renorm ? w_scale / (chosen_sum + 1e-20f) : w_scale;
        for (int r = 0; r < top; ++r) w_out[n * top + r] *= f;
    }
}

// kind 0: silu(g) u;  kind 1: g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit);
// kind 2: no gate, the exact (erf) gelu of u -- the expert's first matrix then has ff rows, not 2 ff
__device__ __forceinline__ float glu_act(float g, float u, int kind, float limit) {
    if (kind == 0) return silu_f(g) * u;
    if (kind == 2) return 0.5f * u * (1.0f + erff(u * 0.7071067811865476f));
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoid_f(1.702f * g) * (u + 1.0f);
}

// The chosen experts of a few tokens.  Every token has `slots` expert calls: its `top` choices and, if there is an always-on
// expert, that one as slot number `top` (table entry n_experts, weight 1).  gate_up[e]: address of expert e's [2 ff_e, width]
// matrix (gate rows first), down[e]: [width, ff_e]; ffs[e] = ff_e (null: `ff` for all).  act: [n_rows, slots, ff] scratch.
// grid (ceil(ff / 8), n_rows * slots), 8 warps a block, one warp per row pair of the gate and up matrices:
// act[n, k, j] = silu(gate_j . h) * (up_j . h).  weight_input: the token's weight for the choice multiplies the expert's INPUT
// (rounded to the model's type) instead of its output
template <typename T>
__global__ void __launch_bounds__(256) moe_small_up_kernel(const T* __restrict__ h, const int32_t* __restrict__ idx, const float* __restrict__ wgt,
                                                           const int64_t* __restrict__ gate_up,
                                                           const int32_t* __restrict__ ffs, int width, int ff, int top, int slots, int n_experts,
                                                           int act_kind, int weight_input, float limit, float limit_always, T* __restrict__ act) {
    const int lane = threadIdx.x & 31;
    const int j = blockIdx.x * 8 + (threadIdx.x >> 5);
    const long nk = blockIdx.y;
    const long n = nk / slots;
    const int k = (int)(nk - n * slots);
    const int e = k < top ? idx[n * top + k] : n_experts;
    if (k < top && e >= n_experts) return;                  // an identity expert, or nothing chosen
    const int ff_e = ffs ? ffs[e] : ff;
    if (j >= ff_e) return;
    const T* w = reinterpret_cast<const T*>(gate_up[e]);
    const T* hr = h + n * width;
    // the products leave the matrix unit of the many-token path rounded to the model's type: the same rounding here
    const bool scaled = weight_input && k < top;
    const float tw = scaled ? wgt[n * top + k] : 1.0f;
    const long up_row = act_kind == 2 ? j : (long)ff_e + j;
    const float g = act_kind == 2 ? 0.0f
                  : to_f(from_f<T>(scaled ? warp_dot_scaled(w + (long)j * width, hr, width, lane, tw) : warp_dot(w + (long)j * width, hr, width, lane)));
    const float u = to_f(from_f<T>(scaled ? warp_dot_scaled(w + up_row * width, hr, width, lane, tw) : warp_dot(w + up_row * width, hr, width, lane)));
    if (lane == 0) act[nk * ff + j] = from_f<T>(glu_act(g, u, act_kind, k < top ? limit : limit_always));
}

// grid (ceil(width / 8), n_rows): one warp per output column.  y[n, c] = sum over the token's slots of w * (down_e[c, :] . act)
// (identity experts: w * h[n, c]) + shared_out[n, c]
template <typename T>
__global__ void __launch_bounds__(256) moe_small_down_kernel(const T* __restrict__ act, const int32_t* __restrict__ idx, const float* __restrict__ wgt,
                                                             const int64_t* __restrict__ down, const int32_t* __restrict__ ffs, const T* __restrict__ h,
                                                             const T* __restrict__ shared_out, int width, int ff, int top, int slots, int n_experts,
                                                             int n_out, const float* __restrict__ always_w, int weight_input, float* __restrict__ y) {
    const int lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + (threadIdx.x >> 5);
    const long n = blockIdx.y;
    if (c >= width) return;
    float sum = 0.0f;
    for (int k = 0; k < slots; ++k) {
        const int e = k < top ? idx[n * top + k] : n_experts;
        const float w = k < top ? (weight_input ? 1.0f : wgt[n * top + k]) : (always_w ? always_w[n] : 1.0f);
        if (k == top || e < n_experts) {
            const int ff_e = ffs ? ffs[e] : ff;
            const T* wd = reinterpret_cast<const T*>(down[e]);
            sum += w * to_f(from_f<T>(warp_dot(wd + (long)c * ff_e, act + (n * slots + k) * ff, ff_e, lane)));
        } else if (e < n_out) {
            sum += wgt[n * top + k] * to_f(h[n * width + c]);
        }
    }
    if (shared_out) sum += to_f(shared_out[n * width + c]);
    if (lane == 0) y[n * width + c] = sum;
}

// Counting sort of the (token, choice) pairs by chosen output, one block: counts[e] = pairs that chose e, pos[i] = row of pair i
// among the pairs sorted by output, token_of[row] = the pair's token.  The order inside one output's rows is whatever the atomic
// counters hand out; every row is computed on its own, so the result does not depend on it.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int32_t* __restrict__ idx, long n_pairs, int top, int n_keys, int32_t* __restrict__ counts,
                                                        int32_t* __restrict__ pos, int64_t* __restrict__ token_of) {
    extern __shared__ int sort_sh[];                        // counts [n_keys], then running offsets [n_keys]
    int* cnt = sort_sh;
    int* off = sort_sh + n_keys;
    for (int e = threadIdx.x; e < n_keys; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (long i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_keys; ++e) { off[e] = run; run += cnt[e]; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_keys; e += blockDim.x) counts[e] = cnt[e];
    for (long i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int p = atomicAdd(&off[idx[i]], 1);
        pos[i] = p;
        token_of[p] = i / top;
    }
}

// rows_in[pos[i], c] = h[i / top, c] * wgt[i] in the model's type, for every (token, choice) pair i that chose an expert: the
// sorted rows of experts that are fed their weighted input
template <typename T>
__global__ void moe_scatter_scaled_kernel(const T* __restrict__ h, const int32_t* __restrict__ pos, const int32_t* __restrict__ idx,
                                          const float* __restrict__ wgt, long n_pairs, int top, int width, int n_experts, T* __restrict__ rows_in) {
    const long total = n_pairs * width;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long pr = i / width;
        const int c = (int)(i - pr * width);
        if (idx[pr] < n_experts) rows_in[(long)pos[pr] * width + c] = from_f<T>(to_f(h[(pr / top) * width + c]) * wgt[pr]);
    }
}

// y[n, c] = sum_k w[n, k] * rows[pos[n, k], c] (identity experts: w * h[n, c]) + shared_w[n] * shared[n, c]; wgt null: weights of 1
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int32_t* __restrict__ pos, const int32_t* __restrict__ idx,
                                   const float* __restrict__ wgt, const T* __restrict__ h, const T* __restrict__ shared_out,
                                   const float* __restrict__ shared_w, long n_rows, int width, int top, int n_experts, int n_out, float* __restrict__ y) {
    const long total = n_rows * width;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long n = i / width;
        const int c = (int)(i - n * width);
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int e = idx[n * top + k];
            const float w = wgt ? wgt[n * top + k] : 1.0f;
            if (e < n_experts) sum += w * to_f(rows[(long)pos[n * top + k] * width + c]);
            else if (e < n_out) sum += w * to_f(h[i]);
        }
        if (shared_out) sum += (shared_w ? shared_w[n] : 1.0f) * to_f(shared_out[i]);
        y[i] = sum;
    }
}

extern "C" int mixers_scored_router(int dtype, const void* h, long n_rows, int width, const void* router, const void* correction, int n_out,
                                    int groups, int keep, int top, int score_mode, int group_top, int renorm, float w_scale,
                                    const void* gate_row, float* gate_out, int32_t* idx_out, float* w_out, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    if (groups < 1 || n_out % groups != 0 || keep < 1 || keep > groups || top < 1 || group_top < 1 || (score_mode != 0 && score_mode != 1) ||
        (gate_row && !gate_out))
        return (int)cudaErrorInvalidValue;
    const int rows = n_out + (gate_row ? 1 : 0);
    int split = 1;                                          // pieces per row: as many as keep every warp busy, none shorter than 512
    while (rows * split * 2 <= ROUTER_WARPS && width / (split * 2) >= 512) split *= 2;
    size_t smem = (size_t)(rows * split + 2 * n_out + groups + ((n_out + groups + 3) / 4)) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const int threads = 32 * (n_rows <= ROUTER_FEW_ROWS ? ROUTER_WARPS : ROUTER_WARPS_MANY);
    MIXERS_DISPATCH(dtype, scored_router_kernel<T><<<(unsigned)n_rows, threads, smem, (cudaStream_t)stream>>>(
        (const T*)h, n_rows, width, (const T*)router, (const T*)correction, n_out, groups, keep, top, score_mode, group_top, renorm, w_scale,
        (const T*)gate_row, gate_out, split, idx_out, w_out));
    return mixers_status();
}

extern "C" int mixers_grouped_router(int dtype, const void* h, long n_rows, int width, const void* router, const void* correction, int n_out,
                                     int groups, int keep, int top, int32_t* idx_out, float* w_out, mixers_stream_t stream) {
    return mixers_scored_router(dtype, h, n_rows, width, router, correction, n_out, groups, keep, top, 0, 1, 0, 1.0f, nullptr, nullptr, idx_out,
                                w_out, stream);
}

extern "C" int mixers_moe_small(int dtype, const void* h, long n_rows, int width, int ff, int top, int n_experts, int n_out, const int32_t* idx,
                                const float* wgt, const int64_t* gate_up, const int64_t* down, const int32_t* ffs, int always_on,
                                const float* always_w, int act_kind, int weight_input, float limit, float limit_always, const void* shared_out,
                                void* act, float* y, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    if (act_kind < 0 || act_kind > 2) return (int)cudaErrorInvalidValue;
    const int slots = top + (always_on ? 1 : 0);
    if (n_rows * slots > 65535 || n_rows > 65535) return (int)cudaErrorInvalidValue;
    if ((n_experts > 0 || always_on) && ff > 0) {
        dim3 g1((ff + 7) / 8, (unsigned)(n_rows * slots));
        MIXERS_DISPATCH(dtype, moe_small_up_kernel<T><<<g1, 256, 0, (cudaStream_t)stream>>>((const T*)h, idx, wgt, gate_up, ffs, width, ff, top, slots,
                                                                                          n_experts, act_kind, weight_input, limit, limit_always,
                                                                                          (T*)act));
    }
    dim3 g2((width + 7) / 8, (unsigned)n_rows);
    MIXERS_DISPATCH(dtype, moe_small_down_kernel<T><<<g2, 256, 0, (cudaStream_t)stream>>>(
        (const T*)act, idx, wgt, down, ffs, (const T*)h, (const T*)shared_out, width, ff, top, slots, n_experts, n_out, always_w, weight_input, y));
    return mixers_status();
}

extern "C" int mixers_moe_combine(int dtype, const void* rows, const int32_t* pos, const int32_t* idx, const float* wgt, const void* h,
                                  const void* shared_out, const float* shared_w, long n_rows, int width, int top, int n_experts, int n_out,
                                  float* y, mixers_stream_t stream) {
    if (n_rows <= 0) return 0;
    long total = n_rows * width;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    MIXERS_DISPATCH(dtype, moe_combine_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const T*)rows, pos, idx, wgt, (const T*)h, (const T*)shared_out, shared_w, n_rows, width, top, n_experts, n_out, y));
    return mixers_status();
}

extern "C" int mixers_moe_sort(const int32_t* idx, long n_pairs, int top, int n_keys, int32_t* counts, int32_t* pos, int64_t* token_of,
                               mixers_stream_t stream) {
    if (n_pairs <= 0) return 0;
    size_t smem = 2 * (size_t)n_keys * sizeof(int);
    if (n_keys < 1 || smem > 48 * 1024 || top < 1) return (int)cudaErrorInvalidValue;
    moe_sort_kernel<<<1, 1024, smem, (cudaStream_t)stream>>>(idx, n_pairs, top, n_keys, counts, pos, token_of);
    return mixers_status();
}

extern "C" int mixers_moe_scatter_scaled(int dtype, const void* h, const int32_t* pos, const int32_t* idx, const float* wgt, long n_pairs, int top,
                                         int width, int n_experts, void* rows_in, mixers_stream_t stream) {
    if (n_pairs <= 0) return 0;
    long blocks = (n_pairs * width + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    MIXERS_DISPATCH(dtype, moe_scatter_scaled_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const T*)h, pos, idx, wgt, n_pairs, top, width,
                                                                                                          n_experts, (T*)rows_in));
    return mixers_status();
}
