// Linear recurrences with a matrix state per head, and the short causal convolution that precedes one of them.
//
// Both recurrences act on every COLUMN of the state independently (a column = one value channel): with M [dim, vdim],
//   gated delta rule:        M <- g M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q
//   gated linear attention:  M <- diag(alpha) M + k v^T;       o = M^T q
//   wkv (RWKV-style):        o = (M + diag(u) k v^T)^T r;      M <- diag(w) M + k v^T     (w = exp(-exp(z + w0)) per key channel)
//   channel delta rule:      M <- diag(a) M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q   (a = exp(-exp(A) softplus(z + bias))
//                                                                                                  per key channel)
//   state-space scan:        M <- g M + dt k v^T;              o = M^T q + D v            (g = exp(-exp(A) dt), dt = softplus(. + bias))
// column j only needs k, q, the token's scalars and v_j.  So a column is owned by LPC lanes of a warp (LPC a power of two), each
// holding R rows of it in registers for the whole call; tokens are taken in order.  Half of the block's warps own columns; the
// other half stage the NEXT 16 tokens meanwhile in the second of two shared-memory buffers: their k / q (/ alpha) rows, scalars
// and v, with unit norms, decays and gates evaluated there in 32-bit floats.
// For the delta rule both dot products are taken on the state BEFORE the token's update,
//   a = M_old^T k,  c = M_old^T q:   u = beta (v - g a),   o = g c + (k . q) u,   M <- g M_old + k u^T,
// which is the same arithmetic reordered so that one round of shuffles serves both.
// The wkv output reads the state BEFORE the token's update plus a bonus for the token itself: o = M_old^T r + (sum_i r_i u_i k_i) v;
// the bonus factor is a scalar per token and head, formed while the token is staged.
#include "mixers_common.cuh"

// one block row per token (blockIdx.x), channels across the block and blockIdx.y: no index division in the loop
// flags: bit 0 = silu on the result, bit 1 = the current token's input is added to the result (y = x + conv(x)); bias may be null
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ proj, int B, int S, int ld, int off, int C, int taps, const T* __restrict__ w,
                                  const T* __restrict__ bias, int flags, const T* __restrict__ tail, T* __restrict__ tail_next, int slot0,
                                  const int32_t* __restrict__ pad, T* __restrict__ y) {
    const int tl = taps - 1 > 0 ? taps - 1 : 1;             // rows of a tail buffer
    const int n = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int b = n / S, t = n - b * S;
    int first = pad ? pad[b] - slot0 : 0;                    // new tokens before this index are padding
    if (first < 0) first = 0;
    const T* in = proj + (long)b * S * ld + off + c;
    const T* tb = tail + (long)b * tl * C + c;
    auto input = [&](int tt) -> float {
        if (tt < 0) return to_f(tb[(long)(taps - 1 + tt) * C]);
        if (tt < first) return 0.0f;
        return to_f(in[(long)tt * ld]);
    };
    float acc = bias ? to_f(bias[c]) : 0.0f;
    for (int j = 0; j < taps; ++j) acc += to_f(w[(long)c * taps + j]) * input(t - (taps - 1) + j);
    if (flags & 1) acc = silu_f(acc);
    if (flags & 2) acc += input(t);
    y[(long)n * C + c] = from_f<T>(t < first ? 0.0f : acc);
    if (t == S - 1)
        for (int r = 0; r < taps - 1; ++r) tail_next[((long)b * tl + r) * C + c] = from_f<T>(input(S - (taps - 1) + r));
}

// Token shift: out[m, n, c] = h[n, c] + (h[n - 1, c] - h[n, c]) * mu[m, c] for each of n_mix mixing vectors; the token before a
// call's first one comes from tail [B, 1, C] (zeros before a sequence's first token), padding slots count as zeros and give
// zeros.  tail_next receives the last token's h (it may be `tail` itself when S == 1: the thread that reads a channel writes it).
template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ h, int B, int S, int C, const T* __restrict__ mu, int n_mix, const T* __restrict__ tail,
                                       T* __restrict__ tail_next, int slot0, const int32_t* __restrict__ pad, T* __restrict__ out) {
    const int n = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int b = n / S, t = n - b * S;
    int first = pad ? pad[b] - slot0 : 0;
    if (first < 0) first = 0;
    const long total = (long)B * S * C;
    const float cur = t < first ? 0.0f : to_f(h[(long)n * C + c]);
    const float before = t == 0 ? to_f(tail[(long)b * C + c]) : (t - 1 < first ? 0.0f : to_f(h[(long)(n - 1) * C + c]));
    for (int m = 0; m < n_mix; ++m)
        out[m * total + (long)n * C + c] = from_f<T>(t < first ? 0.0f : cur + (before - cur) * to_f(mu[(long)m * C + c]));
    if (t == S - 1) tail_next[(long)b * C + c] = from_f<T>(cur);
}

constexpr int REC_CONSUMERS = 128;                          // threads that own state columns (4 warps)
constexpr int REC_PRODUCERS = 128;                          // threads that stage the next tokens meanwhile (4 warps)
constexpr int REC_THREADS = REC_CONSUMERS + REC_PRODUCERS;
constexpr int REC_TPW = 4;                                  // tokens a producer warp stages at a time
constexpr int REC_TC = REC_TPW * (REC_PRODUCERS / 32);      // tokens per stage (16)

// which modes stage a row of decays per token (one per key channel) beside k and q
__host__ __device__ constexpr bool rec_decay_rows(int mode) { return mode == 1 || mode == 2 || mode == 3; }

struct RecArgs {
    const void* src;        // delta: conv output [B, S, C]; gla: projection [B, S, ld]
    int ld_src;
    long off_q, off_k, off_v;  // offsets (elements) of head 0 from the start of a row of src: columns of one projection, or whole
                            // tensors apart when q, k and v are separate [B * S, heads * dim] outputs that follow one another
    int q_heads;            // heads of q / k (delta: kv_heads; gla: heads)
    const void* proj;       // delta: the projection that holds beta / decay logits
    int ld_proj, off_b, off_a;
    const void* A_log;
    const void* dt_bias;
    const void* z;          // gla, wkv, channel delta: decay logits [B, S, heads * dim]
    float inv_tau;
    const void* w0;         // wkv, channel delta: added to the decay logits [heads * dim]
    const void* u;          // wkv: the current token's bonus [heads * dim]; state-space scan: the skip weight D [heads]
    int B, S, heads, dim, vdim, slot0;
    const int32_t* pad;
    float* state;
    float* o;
    int lpc, tc;
};

// shared memory of one stage: k, q (and alpha) rows of tc tokens padded to dp, the block's value columns, three scalars a token
template <int MODE>
struct RecStage {
    float *k, *q, *a, *v, *sc;
    __device__ RecStage(float* base, int tc, int dp, int cols_blk) {
        k = base; q = k + tc * dp; a = q + tc * dp; v = a + (rec_decay_rows(MODE) ? tc * dp : 0); sc = v + tc * cols_blk;
    }
    static __host__ __device__ size_t floats(int tc, int dp, int cols_blk) { return (size_t)tc * ((rec_decay_rows(MODE) ? 3 : 2) * dp + cols_blk + 4); }
};

// producers: tokens t0 .. t0 + nt - 1 of the call into one stage.  A warp takes up to REC_TPW tokens at once, and EVERY global
// load of its share (q, k and decay rows 128 elements at a time, the tokens' scalars one lane each, the first values) is issued
// before the first use of any: a warp issues in order, so each wait on memory would otherwise be paid in full, ~20 times a stage.
template <typename T, int MODE>
__device__ __forceinline__ void rec_stage_tokens(const RecArgs& a, RecStage<MODE> st, int b, int h, int qh, int t0, int nt, int dp, int cols_blk,
                                                 int col0, int ptid, float neg_exp_a, float dt_bias) {
    const int lane = ptid & 31, pw = ptid >> 5;
    const int dim = a.dim, S = a.S;
    const T* src = (const T*)a.src;
    const float q_scale = rsqrtf((float)dim);
    const int tt0 = pw * REC_TPW;
    int cnt = nt - tt0;
    if (cnt > REC_TPW) cnt = REC_TPW;
    // the block's value columns: the first (usually only) batch of loads goes out now and is stored at the end
    constexpr int VB = 4;
    const int nv = nt * cols_blk;
    float vreg[VB];
#pragma unroll
    for (int e = 0; e < VB; ++e) {
        int i = ptid + e * REC_PRODUCERS;
        vreg[e] = 0.0f;
        if (i < nv) {
            int tt = i / cols_blk, cg = col0 + (i - tt * cols_blk);
            if (cg < a.vdim) vreg[e] = to_f(src[((long)b * S + t0 + tt) * a.ld_src + a.off_v + h * a.vdim + cg]);
        }
    }
    float lb = 0.0f, la = 0.0f;                              // lane j: the gate logits of the warp's token j
    if ((MODE == 0 || MODE == 3 || MODE == 4) && lane < cnt) {
        const T* pr = (const T*)a.proj + ((long)b * S + t0 + tt0 + lane) * a.ld_proj;
        if (MODE != 4) lb = to_f(pr[a.off_b + h]);
        if (MODE != 3) la = to_f(pr[a.off_a + h]);
    }
    if (cnt > 0) {
        float sq[REC_TPW], sk[REC_TPW], skq[REC_TPW];
#pragma unroll
        for (int j = 0; j < REC_TPW; ++j) sq[j] = sk[j] = skq[j] = 0.0f;
        for (int blk = 0; blk < dp; blk += 128) {
            float qv[REC_TPW][4], kv[REC_TPW][4], zv[REC_TPW][4], w0v[4], uv[4];
            if (MODE == 2 || MODE == 3) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = blk + lane + 32 * e;
                    w0v[e] = i < dim ? to_f(((const T*)a.w0)[h * dim + i]) : 0.0f;
                    if (MODE == 2) uv[e] = i < dim ? to_f(((const T*)a.u)[h * dim + i]) : 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < REC_TPW; ++j) {
                const T* row = src + ((long)b * S + t0 + tt0 + (j < cnt ? j : 0)) * a.ld_src;
                const T* zr = rec_decay_rows(MODE) ? (const T*)a.z + ((long)b * S + t0 + tt0 + (j < cnt ? j : 0)) * ((long)a.heads * dim) + h * dim : nullptr;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = blk + lane + 32 * e;
                    const bool ok = j < cnt && i < dim;
                    qv[j][e] = ok ? to_f(row[a.off_q + qh * dim + i]) : 0.0f;
                    kv[j][e] = ok ? to_f(row[a.off_k + qh * dim + i]) : 0.0f;
                    if (rec_decay_rows(MODE)) zv[j][e] = ok ? to_f(zr[i]) : 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < REC_TPW; ++j) {
                if (j < cnt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = blk + lane + 32 * e;
                        if (i < dp) {
                            if (MODE == 1) {
                                st.a[(tt0 + j) * dp + i] = i < dim ? expf(log_sigmoid_f(zv[j][e]) * a.inv_tau) : 1.0f;
                                st.q[(tt0 + j) * dp + i] = qv[j][e] * q_scale;
                            } else if (MODE == 2) {
                                st.a[(tt0 + j) * dp + i] = i < dim ? expf(-expf(zv[j][e] + w0v[e])) : 1.0f;
                                st.q[(tt0 + j) * dp + i] = qv[j][e];
                                skq[j] += qv[j][e] * uv[e] * kv[j][e];
                            } else if (MODE == 4) {
                                st.q[(tt0 + j) * dp + i] = qv[j][e];
                            } else {
                                if (MODE == 3) st.a[(tt0 + j) * dp + i] = i < dim ? expf(neg_exp_a * softplus_f(zv[j][e] + w0v[e])) : 1.0f;
                                st.q[(tt0 + j) * dp + i] = qv[j][e];
                                sq[j] += qv[j][e] * qv[j][e]; sk[j] += kv[j][e] * kv[j][e]; skq[j] += qv[j][e] * kv[j][e];
                            }
                            st.k[(tt0 + j) * dp + i] = kv[j][e];
                        }
                    }
                }
            }
        }
        if (MODE == 0 || MODE == 3) {
#pragma unroll
            for (int j = 0; j < REC_TPW; ++j) { sq[j] = warp_sum(sq[j]); sk[j] = warp_sum(sk[j]); skq[j] = warp_sum(skq[j]); }
            __syncwarp();
            float my_nq = 0.0f, my_nk = 0.0f, my_kq = 0.0f;
#pragma unroll
            for (int j = 0; j < REC_TPW; ++j) {
                if (j < cnt) {
                    const float nq = q_scale / sqrtf(sq[j] + 1e-6f), nk = 1.0f / sqrtf(sk[j] + 1e-6f);
                    for (int i = lane; i < dp; i += 32) { st.q[(tt0 + j) * dp + i] *= nq; st.k[(tt0 + j) * dp + i] *= nk; }
                    if (lane == j) { my_nq = nq; my_nk = nk; my_kq = skq[j]; }
                }
            }
            if (lane < cnt) {
                st.sc[(tt0 + lane) * 4 + 0] = MODE == 0 ? expf(neg_exp_a * softplus_f(la + dt_bias)) : 1.0f;
                st.sc[(tt0 + lane) * 4 + 1] = sigmoid_f(lb);
                st.sc[(tt0 + lane) * 4 + 2] = my_kq * my_nq * my_nk;
            }
        }
        if (MODE == 4 && lane < cnt) {
            const float dt = softplus_f(la + dt_bias);
            st.sc[(tt0 + lane) * 4 + 0] = expf(neg_exp_a * dt);
            st.sc[(tt0 + lane) * 4 + 1] = dt;
        }
        if (MODE == 2) {
            float mine = 0.0f;
#pragma unroll
            for (int j = 0; j < REC_TPW; ++j) { const float tot = warp_sum(skq[j]); if (lane == j) mine = tot; }
            if (lane < cnt) st.sc[(tt0 + lane) * 4 + 2] = mine;
        }
    }
#pragma unroll
    for (int e = 0; e < VB; ++e) {
        int i = ptid + e * REC_PRODUCERS;
        if (i < nv) st.v[i] = vreg[e];
    }
    for (int i = ptid + VB * REC_PRODUCERS; i < nv; i += REC_PRODUCERS) {          // narrow heads only: more columns than one batch
        int tt = i / cols_blk, cg = col0 + (i - tt * cols_blk);
        st.v[i] = cg < a.vdim ? to_f(src[((long)b * S + t0 + tt) * a.ld_src + a.off_v + h * a.vdim + cg]) : 0.0f;
    }
}

// MINB: blocks that must fit an SM together.  0 (no demand) leaves the choice of registers to the compiler (a grid of at most
// one block per SM: what counts is how fast ONE block walks its tokens; demanding 1 explicitly made it take more registers and
// run 10 % slower); 2 halves them (some spills) so that two blocks hide each other's latencies, which pays when the grid has
// more blocks than the GPU has SMs (batches, many heads): measured for the wkv mode only.
template <typename T, int MODE, int R, int MINB>           // MODE 0: gated delta rule, 1: gated linear attention, 2: wkv,
                                                           // 3: channel delta rule, 4: state-space scan
__global__ void __launch_bounds__(REC_THREADS, MINB) linear_recurrence_kernel(RecArgs a) {
    extern __shared__ float sh[];
    const int lpc = a.lpc, dp = R * lpc, tc = a.tc;
    const int cols_blk = REC_CONSUMERS / lpc;
    const size_t stage_floats = RecStage<MODE>::floats(tc, dp, cols_blk);
    const int b = blockIdx.z, h = blockIdx.y;
    const int tid = threadIdx.x;
    const bool producer = tid >= REC_CONSUMERS;
    const int sub = tid % lpc;                               // consumers only
    const int col_l = tid / lpc;
    const int col0 = blockIdx.x * cols_blk;
    const int col = col0 + col_l;
    const bool col_ok = !producer && col < a.vdim;
    const int dim = a.dim, vdim = a.vdim, S = a.S;
    const int qh = h / (a.heads / a.q_heads);

    float M[R];
    float* stp = a.state + ((long)b * a.heads + h) * dim * vdim;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int i = r * lpc + sub;
        M[r] = (col_ok && i < dim) ? stp[(long)i * vdim + col] : 0.0f;
    }
    int first = a.pad ? a.pad[b] - a.slot0 : 0;
    if (first < 0) first = 0;
    if (first > S) first = S;
    float* obase = a.o + (((long)b * S) * a.heads + h) * vdim;
    if (sub == 0 && col_ok)
        for (int t = 0; t < first; ++t) obase[(long)t * a.heads * vdim + col] = 0.0f;

    const int nchunks = (S - first + tc - 1) / tc;
    float neg_exp_a = 0.0f, dt_bias = 0.0f;
    if ((MODE == 0 || MODE == 3 || MODE == 4) && producer) {
        neg_exp_a = -expf(to_f(((const T*)a.A_log)[h]));
        if (MODE != 3) dt_bias = to_f(((const T*)a.dt_bias)[h]);
    }
    const float skip = (MODE == 4 && !producer) ? to_f(((const T*)a.u)[h]) : 0.0f;
    if (producer && nchunks > 0)
        rec_stage_tokens<T, MODE>(a, RecStage<MODE>(sh, tc, dp, cols_blk), b, h, qh, first, (S - first < tc ? S - first : tc), dp, cols_blk, col0,
                                  tid - REC_CONSUMERS, neg_exp_a, dt_bias);
    __syncthreads();
    for (int ci = 0; ci < nchunks; ++ci) {
        const int t0 = first + ci * tc;
        if (producer) {
            if (ci + 1 < nchunks) {
                const int t1 = t0 + tc;
                rec_stage_tokens<T, MODE>(a, RecStage<MODE>(sh + ((ci + 1) & 1) * stage_floats, tc, dp, cols_blk), b, h, qh, t1,
                                          (S - t1 < tc ? S - t1 : tc), dp, cols_blk, col0, tid - REC_CONSUMERS, neg_exp_a, dt_bias);
            }
        } else {
            // the tokens in order; a column's lanes only talk to each other.  Four partial sums per dot product keep the
            // dependent chains short.
            const RecStage<MODE> st(sh + (ci & 1) * stage_floats, tc, dp, cols_blk);
            const int nt = S - t0 < tc ? S - t0 : tc;
            for (int tt = 0; tt < nt; ++tt) {
                const float* kk = st.k + tt * dp + sub;
                const float* qq = st.q + tt * dp + sub;
                const float v = st.v[tt * cols_blk + col_l];
                float kr[R], qr[R];
#pragma unroll
                for (int r = 0; r < R; ++r) { kr[r] = kk[r * lpc]; qr[r] = qq[r * lpc]; }
                float o;
                if (MODE == 0) {
                    const float g = st.sc[tt * 4 + 0], beta = st.sc[tt * 4 + 1], kq = st.sc[tt * 4 + 2];
                    float ak[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int r = 0; r < R; ++r) { ak[r & 3] += M[r] * kr[r]; cq[r & 3] += M[r] * qr[r]; }
                    float aks = (ak[0] + ak[1]) + (ak[2] + ak[3]), cqs = (cq[0] + cq[1]) + (cq[2] + cq[3]);
#pragma unroll
                    for (int r = 0; r < R; ++r) M[r] *= g;                   // overlaps the shuffles below
                    for (int m = lpc >> 1; m > 0; m >>= 1) { aks += __shfl_xor_sync(0xffffffffu, aks, m); cqs += __shfl_xor_sync(0xffffffffu, cqs, m); }
                    const float u = beta * (v - g * aks);
                    o = g * cqs + kq * u;
#pragma unroll
                    for (int r = 0; r < R; ++r) M[r] += kr[r] * u;
                } else if (MODE == 3) {
                    const float* aa = st.a + tt * dp + sub;
                    const float beta = st.sc[tt * 4 + 1], kq = st.sc[tt * 4 + 2];
                    float ak[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int r = 0; r < R; ++r) { M[r] *= aa[r * lpc]; ak[r & 3] += M[r] * kr[r]; cq[r & 3] += M[r] * qr[r]; }
                    float aks = (ak[0] + ak[1]) + (ak[2] + ak[3]), cqs = (cq[0] + cq[1]) + (cq[2] + cq[3]);
                    for (int m = lpc >> 1; m > 0; m >>= 1) { aks += __shfl_xor_sync(0xffffffffu, aks, m); cqs += __shfl_xor_sync(0xffffffffu, cqs, m); }
                    const float u = beta * (v - aks);
                    o = cqs + kq * u;
#pragma unroll
                    for (int r = 0; r < R; ++r) M[r] += kr[r] * u;
                } else if (MODE == 4) {
                    const float g = st.sc[tt * 4 + 0], dv = st.sc[tt * 4 + 1] * v;
                    float op[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int r = 0; r < R; ++r) { M[r] = g * M[r] + kr[r] * dv; op[r & 3] += M[r] * qr[r]; }
                    o = (op[0] + op[1]) + (op[2] + op[3]);
                    for (int m = lpc >> 1; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
                    o += skip * v;
                } else if (MODE == 1) {
                    const float* aa = st.a + tt * dp + sub;
                    float op[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int r = 0; r < R; ++r) { M[r] = aa[r * lpc] * M[r] + kr[r] * v; op[r & 3] += M[r] * qr[r]; }
                    o = (op[0] + op[1]) + (op[2] + op[3]);
                    for (int m = lpc >> 1; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
                } else {
                    const float* aa = st.a + tt * dp + sub;
                    float op[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int r = 0; r < R; ++r) { op[r & 3] += M[r] * qr[r]; M[r] = aa[r * lpc] * M[r] + kr[r] * v; }
                    o = (op[0] + op[1]) + (op[2] + op[3]);
                    for (int m = lpc >> 1; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
                    o += st.sc[tt * 4 + 2] * v;
                }
                if (sub == 0 && col_ok) obase[(long)(t0 + tt) * a.heads * vdim + col] = o;
            }
        }
        __syncthreads();
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = r * lpc + sub;
            if (i < dim) stp[(long)i * vdim + col] = M[r];
        }
    }
}

// ---- a few new tokens (decoding, short portions): no pipeline to fill.  The whole block stages up to tc tokens, then every
// thread runs them on its rows of its column; 128 threads and half the registers of the pipelined kernel, so that the
// many small blocks of a decode step (batch x heads x column blocks) are resident together.
constexpr int REC_FEW_THREADS = 128;

template <typename T, int MODE, int R>
__global__ void __launch_bounds__(REC_FEW_THREADS) linear_recurrence_few_kernel(RecArgs a) {
    extern __shared__ float sh[];
    const int lpc = a.lpc, dp = R * lpc, tc = a.tc;
    const int cols_blk = REC_FEW_THREADS / lpc;
    float* kbuf = sh;                                        // [tc][dp]
    float* qbuf = kbuf + tc * dp;                            // [tc][dp]
    float* abuf = qbuf + tc * dp;                            // [tc][dp] (gla, wkv)
    float* vbuf = abuf + (rec_decay_rows(MODE) ? tc * dp : 0);   // [tc][cols_blk]
    float* sc = vbuf + tc * cols_blk;                        // [tc][4]: g, beta, k.q (wkv: [2] = sum r u k)
    const int b = blockIdx.z, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int sub = tid % lpc;
    const int col_l = tid / lpc;
    const int col = blockIdx.x * cols_blk + col_l;
    const bool col_ok = col < a.vdim;
    const int dim = a.dim, vdim = a.vdim, S = a.S;
    const int qh = h / (a.heads / a.q_heads);
    const T* src = (const T*)a.src;

    float M[R];
    float* st = a.state + ((long)b * a.heads + h) * dim * vdim;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int i = r * lpc + sub;
        M[r] = (col_ok && i < dim) ? st[(long)i * vdim + col] : 0.0f;
    }
    int first = a.pad ? a.pad[b] - a.slot0 : 0;
    if (first < 0) first = 0;
    if (first > S) first = S;
    float* obase = a.o + (((long)b * S) * a.heads + h) * vdim;
    if (sub == 0 && col_ok)
        for (int t = 0; t < first; ++t) obase[(long)t * a.heads * vdim + col] = 0.0f;
    const float q_scale = rsqrtf((float)dim);
    const float skip = MODE == 4 ? to_f(((const T*)a.u)[h]) : 0.0f;

    for (int t0 = first; t0 < S; t0 += tc) {
        const int nt = S - t0 < tc ? S - t0 : tc;
        __syncthreads();
        // ---- stage nt tokens: a warp per token
        for (int tt = wid; tt < nt; tt += REC_FEW_THREADS / 32) {
            const T* row = src + ((long)b * S + t0 + tt) * a.ld_src;
            const T* qr = row + a.off_q + qh * dim;
            const T* kr = row + a.off_k + qh * dim;
            float sq = 0.0f, sk = 0.0f, skq = 0.0f;
            for (int i = lane; i < dp; i += 32) {
                float qv = i < dim ? to_f(qr[i]) : 0.0f, kv = i < dim ? to_f(kr[i]) : 0.0f;
                qbuf[tt * dp + i] = qv;
                kbuf[tt * dp + i] = kv;
                sq += qv * qv; sk += kv * kv; skq += qv * kv;
            }
            if (MODE == 0 || MODE == 3) {
                sq = warp_sum(sq); sk = warp_sum(sk); skq = warp_sum(skq);
                const float nq = q_scale / sqrtf(sq + 1e-6f), nk = 1.0f / sqrtf(sk + 1e-6f);
                __syncwarp();
                for (int i = lane; i < dp; i += 32) { qbuf[tt * dp + i] *= nq; kbuf[tt * dp + i] *= nk; }
                if (MODE == 3) {
                    const T* zr = (const T*)a.z + ((long)b * S + t0 + tt) * ((long)a.heads * dim) + h * dim;
                    const T* w0 = (const T*)a.w0 + h * dim;
                    const float neg_exp_a = -expf(to_f(((const T*)a.A_log)[h]));
                    for (int i = lane; i < dp; i += 32) abuf[tt * dp + i] = i < dim ? expf(neg_exp_a * softplus_f(to_f(zr[i]) + to_f(w0[i]))) : 1.0f;
                }
                if (lane == 0) {
                    const T* pr = (const T*)a.proj + ((long)b * S + t0 + tt) * a.ld_proj;
                    float beta = sigmoid_f(to_f(pr[a.off_b + h]));
                    if (MODE == 0) {
                        float dt = softplus_f(to_f(pr[a.off_a + h]) + to_f(((const T*)a.dt_bias)[h]));
                        sc[tt * 4 + 0] = expf(-expf(to_f(((const T*)a.A_log)[h])) * dt);
                    }
                    sc[tt * 4 + 1] = beta;
                    sc[tt * 4 + 2] = skq * nq * nk;
                }
            } else if (MODE == 4) {
                if (lane == 0) {
                    const T* pr = (const T*)a.proj + ((long)b * S + t0 + tt) * a.ld_proj;
                    const float dt = softplus_f(to_f(pr[a.off_a + h]) + to_f(((const T*)a.dt_bias)[h]));
                    sc[tt * 4 + 0] = expf(-expf(to_f(((const T*)a.A_log)[h])) * dt);
                    sc[tt * 4 + 1] = dt;
                }
            } else if (MODE == 1) {
                const T* zr = (const T*)a.z + ((long)b * S + t0 + tt) * ((long)a.heads * dim) + h * dim;
                for (int i = lane; i < dp; i += 32) {
                    qbuf[tt * dp + i] *= q_scale;
                    abuf[tt * dp + i] = i < dim ? expf(log_sigmoid_f(to_f(zr[i])) * a.inv_tau) : 1.0f;
                }
            } else {
                const T* zr = (const T*)a.z + ((long)b * S + t0 + tt) * ((long)a.heads * dim) + h * dim;
                const T* w0 = (const T*)a.w0 + h * dim;
                const T* uu = (const T*)a.u + h * dim;
                float ruk = 0.0f;
                for (int i = lane; i < dp; i += 32) {
                    abuf[tt * dp + i] = i < dim ? expf(-expf(to_f(zr[i]) + to_f(w0[i]))) : 1.0f;
                    if (i < dim) ruk += qbuf[tt * dp + i] * to_f(uu[i]) * kbuf[tt * dp + i];
                }
                ruk = warp_sum(ruk);
                if (lane == 0) sc[tt * 4 + 2] = ruk;
            }
        }
        for (int i = tid; i < nt * cols_blk; i += REC_FEW_THREADS) {
            int tt = i / cols_blk, cl = i - tt * cols_blk;
            int cg = blockIdx.x * cols_blk + cl;
            vbuf[i] = cg < vdim ? to_f(src[((long)b * S + t0 + tt) * a.ld_src + a.off_v + h * vdim + cg]) : 0.0f;
        }
        __syncthreads();
        // ---- the tokens in order; a column's lanes only talk to each other
        for (int tt = 0; tt < nt; ++tt) {
            const float* kk = kbuf + tt * dp + sub;
            const float* qq = qbuf + tt * dp + sub;
            const float v = vbuf[tt * cols_blk + col_l];
            float o;
            if (MODE == 0) {
                float ak = 0.0f, cq = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) { ak += M[r] * kk[r * lpc]; cq += M[r] * qq[r * lpc]; }
                for (int m = lpc >> 1; m > 0; m >>= 1) { ak += __shfl_xor_sync(0xffffffffu, ak, m); cq += __shfl_xor_sync(0xffffffffu, cq, m); }
                const float g = sc[tt * 4 + 0], beta = sc[tt * 4 + 1], kq = sc[tt * 4 + 2];
                const float u = beta * (v - g * ak);
                o = g * cq + kq * u;
#pragma unroll
                for (int r = 0; r < R; ++r) M[r] = g * M[r] + kk[r * lpc] * u;
            } else if (MODE == 3) {
                const float* aa = abuf + tt * dp + sub;
                float ak = 0.0f, cq = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) { M[r] *= aa[r * lpc]; ak += M[r] * kk[r * lpc]; cq += M[r] * qq[r * lpc]; }
                for (int m = lpc >> 1; m > 0; m >>= 1) { ak += __shfl_xor_sync(0xffffffffu, ak, m); cq += __shfl_xor_sync(0xffffffffu, cq, m); }
                const float u = sc[tt * 4 + 1] * (v - ak);
                o = cq + sc[tt * 4 + 2] * u;
#pragma unroll
                for (int r = 0; r < R; ++r) M[r] += kk[r * lpc] * u;
            } else if (MODE == 4) {
                const float g = sc[tt * 4 + 0], dv = sc[tt * 4 + 1] * v;
                o = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) { M[r] = g * M[r] + kk[r * lpc] * dv; o += M[r] * qq[r * lpc]; }
                for (int m = lpc >> 1; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
                o += skip * v;
            } else if (MODE == 1) {
                const float* aa = abuf + tt * dp + sub;
                o = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) { M[r] = aa[r * lpc] * M[r] + kk[r * lpc] * v; o += M[r] * qq[r * lpc]; }
                for (int m = lpc >> 1; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
            } else {
                const float* aa = abuf + tt * dp + sub;
                o = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) { o += M[r] * qq[r * lpc]; M[r] = aa[r * lpc] * M[r] + kk[r * lpc] * v; }
                for (int m = lpc >> 1; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
                o += sc[tt * 4 + 2] * v;
            }
            if (sub == 0 && col_ok) obase[(long)(t0 + tt) * a.heads * vdim + col] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = r * lpc + sub;
            if (i < dim) st[(long)i * vdim + col] = M[r];
        }
    }
}


template <typename T, int MODE>
static int launch_recurrence_few(RecArgs a, cudaStream_t stream) {
    int r = a.dim <= 512 ? 16 : 32;
    int need = (a.dim + r - 1) / r;
    int lpc = 1;
    while (lpc < need) lpc <<= 1;
    if (lpc > 32) return (int)cudaErrorInvalidValue;
    int dp = r * lpc, cols_blk = REC_FEW_THREADS / lpc;
    int arrays = rec_decay_rows(MODE) ? 3 : 2;
    int tc = a.S < REC_TC ? a.S : REC_TC;
    auto bytes = [&](int n) { return (size_t)n * (arrays * dp + cols_blk + 4) * sizeof(float); };
    while (tc > 1 && bytes(tc) > 40 * 1024) tc >>= 1;
    if (bytes(tc) > 48 * 1024) return (int)cudaErrorInvalidValue;
    a.lpc = lpc; a.tc = tc;
    dim3 grid((a.vdim + cols_blk - 1) / cols_blk, a.heads, a.B);
    if (r == 16) linear_recurrence_few_kernel<T, MODE, 16><<<grid, REC_FEW_THREADS, bytes(tc), stream>>>(a);
    else linear_recurrence_few_kernel<T, MODE, 32><<<grid, REC_FEW_THREADS, bytes(tc), stream>>>(a);
    return mixers_status();
}

template <typename T, int MODE>
static int launch_recurrence(RecArgs a, cudaStream_t stream) {
    if (a.S < REC_TC) return launch_recurrence_few<T, MODE>(a, stream);        // less than one stage of tokens
    int r = a.dim <= 512 ? 16 : 32;
    int need = (a.dim + r - 1) / r;
    int lpc = 1;
    while (lpc < need) lpc <<= 1;
    if (lpc > 32) return (int)cudaErrorInvalidValue;         // heads wider than 1024 rows are not served
    int dp = r * lpc, cols_blk = REC_CONSUMERS / lpc;
    size_t bytes = 2 * RecStage<MODE>::floats(REC_TC, dp, cols_blk) * sizeof(float);      // two stages
    if (bytes > 160 * 1024) return launch_recurrence_few<T, MODE>(a, stream);  // very wide heads: stages of fewer tokens, unpipelined
    a.lpc = lpc; a.tc = REC_TC;
    dim3 grid((a.vdim + cols_blk - 1) / cols_blk, a.heads, a.B);
    const bool pair = (MODE == 2 || MODE == 3) && (long)grid.x * grid.y * grid.z > 148 && 2 * bytes <= 200 * 1024;
    auto kernel = r == 16 ? (pair ? linear_recurrence_kernel<T, MODE, 16, 2> : linear_recurrence_kernel<T, MODE, 16, 0>)
                          : (pair ? linear_recurrence_kernel<T, MODE, 32, 2> : linear_recurrence_kernel<T, MODE, 32, 0>);
    static size_t allowed[4] = {48 * 1024, 48 * 1024, 48 * 1024, 48 * 1024};   // per instantiation: raised once, outside any capture
    size_t& cur = allowed[(r == 16 ? 0 : 1) + (pair ? 2 : 0)];
    if (bytes > cur) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        cur = 200 * 1024;
    }
    kernel<<<grid, REC_THREADS, bytes, stream>>>(a);
    return mixers_status();
}

extern "C" int mixers_short_conv(int dtype, const void* proj, int B, int S, int ld, int off, int C, int taps, const void* w, const void* bias,
                                 int flags, const void* tail, void* tail_next, int slot0, const int32_t* pad, void* y, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (taps < 1 || (flags & ~3)) return (int)cudaErrorInvalidValue;
    const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
    dim3 blocks((unsigned)((long)B * S), (unsigned)((C + threads - 1) / threads));
    MIXERS_DISPATCH(dtype, short_conv_kernel<T><<<blocks, threads, 0, (cudaStream_t)stream>>>((const T*)proj, B, S, ld, off, C, taps, (const T*)w,
                                                                                            (const T*)bias, flags, (const T*)tail, (T*)tail_next, slot0,
                                                                                            pad, (T*)y));
    return mixers_status();
}

extern "C" int mixers_short_conv_silu(int dtype, const void* proj, int B, int S, int ld, int off, int C, int taps, const void* w,
                                      const void* tail, void* tail_next, int slot0, const int32_t* pad, void* y, mixers_stream_t stream) {
    return mixers_short_conv(dtype, proj, B, S, ld, off, C, taps, w, nullptr, 1, tail, tail_next, slot0, pad, y, stream);
}

extern "C" int mixers_token_shift_mix(int dtype, const void* h, int B, int S, int C, const void* mu, int n_mix, const void* tail, void* tail_next,
                                      int slot0, const int32_t* pad, void* out, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
    dim3 blocks((unsigned)((long)B * S), (unsigned)((C + threads - 1) / threads));
    MIXERS_DISPATCH(dtype, token_shift_mix_kernel<T><<<blocks, threads, 0, (cudaStream_t)stream>>>((const T*)h, B, S, C, (const T*)mu, n_mix, (const T*)tail,
                                                                                                 (T*)tail_next, slot0, pad, (T*)out));
    return mixers_status();
}

extern "C" int mixers_gated_delta_rule(int dtype, const void* conv, int B, int S, int kv_heads, int heads, int dim, int vdim,
                                       const void* proj, int ld, int off_b, int off_a, const void* A_log, const void* dt_bias, float* state,
                                       int slot0, const int32_t* pad, float* o, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
    RecArgs a = {};
    a.src = conv; a.ld_src = 2 * kv_heads * dim + heads * vdim;
    a.off_q = 0; a.off_k = kv_heads * dim; a.off_v = 2 * kv_heads * dim; a.q_heads = kv_heads;
    a.proj = proj; a.ld_proj = ld; a.off_b = off_b; a.off_a = off_a; a.A_log = A_log; a.dt_bias = dt_bias;
    a.B = B; a.S = S; a.heads = heads; a.dim = dim; a.vdim = vdim; a.slot0 = slot0; a.pad = pad; a.state = state; a.o = o;
    MIXERS_DISPATCH(dtype, return (launch_recurrence<T, 0>(a, (cudaStream_t)stream)));
    return 0;
}

extern "C" int mixers_gated_linear_attention(int dtype, const void* proj, int B, int S, int ld, int heads, int dim, int vdim, const void* z,
                                             float tau, float* state, int slot0, const int32_t* pad, float* o, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    RecArgs a = {};
    a.src = proj; a.ld_src = ld; a.off_q = 0; a.off_k = heads * dim; a.off_v = 2 * heads * dim; a.q_heads = heads;
    a.z = z; a.inv_tau = 1.0f / tau;
    a.B = B; a.S = S; a.heads = heads; a.dim = dim; a.vdim = vdim; a.slot0 = slot0; a.pad = pad; a.state = state; a.o = o;
    MIXERS_DISPATCH(dtype, return (launch_recurrence<T, 1>(a, (cudaStream_t)stream)));
    return 0;
}

extern "C" int mixers_wkv(int dtype, const void* r, const void* k, const void* v, int B, int S, int ld, int heads, int dim, const void* z,
                          const void* w0, const void* u, float* state, int slot0, const int32_t* pad, float* o, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    const long esz = dtype == 0 ? 4 : 2;
    RecArgs a = {};
    a.src = r; a.ld_src = ld; a.off_q = 0;
    a.off_k = (long)(((const char*)k - (const char*)r) / esz); a.off_v = (long)(((const char*)v - (const char*)r) / esz);
    a.q_heads = heads; a.z = z; a.w0 = w0; a.u = u;
    a.B = B; a.S = S; a.heads = heads; a.dim = dim; a.vdim = dim; a.slot0 = slot0; a.pad = pad; a.state = state; a.o = o;
    MIXERS_DISPATCH(dtype, return (launch_recurrence<T, 2>(a, (cudaStream_t)stream)));
    return 0;
}

extern "C" int mixers_channel_delta_rule(int dtype, const void* conv, int B, int S, int kv_heads, int heads, int dim, int vdim, const void* proj,
                                         int ld, int off_b, const void* z, const void* A_log, const void* dt_bias, float* state, int slot0,
                                         const int32_t* pad, float* o, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (kv_heads < 1 || heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
    RecArgs a = {};
    a.src = conv; a.ld_src = 2 * kv_heads * dim + heads * vdim;
    a.off_q = 0; a.off_k = kv_heads * dim; a.off_v = 2 * kv_heads * dim; a.q_heads = kv_heads;
    a.proj = proj; a.ld_proj = ld; a.off_b = off_b; a.z = z; a.A_log = A_log; a.w0 = dt_bias;
    a.B = B; a.S = S; a.heads = heads; a.dim = dim; a.vdim = vdim; a.slot0 = slot0; a.pad = pad; a.state = state; a.o = o;
    MIXERS_DISPATCH(dtype, return (launch_recurrence<T, 3>(a, (cudaStream_t)stream)));
    return 0;
}

extern "C" int mixers_state_space_scan(int dtype, const void* conv, int B, int S, int groups, int heads, int n_state, int vdim, const void* proj,
                                       int ld, int off_dt, const void* A_log, const void* dt_bias, const void* skip, float* state, int slot0,
                                       const int32_t* pad, float* o, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (groups < 1 || heads % groups != 0) return (int)cudaErrorInvalidValue;
    RecArgs a = {};
    a.src = conv; a.ld_src = heads * vdim + 2 * groups * n_state;
    a.off_v = 0; a.off_k = heads * vdim; a.off_q = heads * vdim + groups * n_state; a.q_heads = groups;
    a.proj = proj; a.ld_proj = ld; a.off_a = off_dt; a.A_log = A_log; a.dt_bias = dt_bias; a.u = skip;
    a.B = B; a.S = S; a.heads = heads; a.dim = n_state; a.vdim = vdim; a.slot0 = slot0; a.pad = pad; a.state = state; a.o = o;
    MIXERS_DISPATCH(dtype, return (launch_recurrence<T, 4>(a, (cudaStream_t)stream)));
    return 0;
}
