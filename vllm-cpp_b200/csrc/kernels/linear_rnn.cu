// Recurrent mixers whose state is a matrix per head, S [d][dv] in 32-bit, carried from token to token in the request's slot:
//
//  * the gated delta rule    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                            q, k: the head's rows of a convolved buffer, made unit vectors here (x / sqrt(sum x^2 + 1e-6)),
//                            q times d^(-1/2); beta = sigmoid(b); g = exp(-rate_h softplus(a + dt_bias_h))
//  * the gated linear form   S <- diag(f) S + (1 - f) v^T;  o = S^T q
//                            q = silu(.), f = low + (1 - low) sigmoid(. + bias), all from one row of 32-bit sums
//  * head_norm_gate          every head of o divided by its root mean square, times a gain shared by the heads, times
//                            silu(gate) where there is a gate
//
// One token after the other is the only order the recurrences allow.  A block owns (entry, head, a tile of value columns):
// a column's d state rows lie in the registers of L neighbouring lanes (R rows each), whose partial sums meet in shuffles;
// the inputs of eight tokens are staged in shared memory at a time, so the token loop itself has no barrier.  The order of
// every sum depends on d only, never on how a prompt was cut: a cut changes nothing but the place of the barrier.
#include "common.cuh"

namespace {

constexpr int R = 16;          // state rows a thread keeps
constexpr int TB = 8;          // tokens staged at a time
constexpr int THREADS = 256;

struct Rows {
    const float* p;
    int S;
    long long s_stride;
    long long ld;
};

__device__ __forceinline__ float rows_at(const Rows& in, long long t, int c) {
    float v = 0.f;
    const float* p = in.p + t * in.ld + c;
    for (int s = 0; s < in.S; ++s) v += p[(long long)s * in.s_stride];
    return v;
}

__device__ __forceinline__ int entry_of_row(const int* __restrict__ q_start, const int* __restrict__ q_len, int E, int t) {
    int lo = 0, hi = E;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (q_start[mid] <= t) lo = mid + 1;
        else hi = mid;
    }
    const int e = lo - 1;
    if (e < 0) return -1;
    return t - q_start[e] < q_len[e] ? e : -1;
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

enum { MODE_DELTA = 0, MODE_GATED = 1 };

struct RnnArgs {
    Rows u;                 // the projection's sums
    const float* x;         // MODE_DELTA: the convolved q | k | v rows [T][ldx], 32-bit
    long long ldx;
    int q_col, k_col, v_col;        // first column of q, of k (MODE_GATED: of the forget gate's sums), of v -- q, k in x
                                    // (MODE_DELTA) or u (MODE_GATED), v likewise
    int b_col, a_col;       // MODE_DELTA: columns of u with beta's and the decay's sums, one per head
    const float* dt_bias;   // [H]
    const float* rate;      // [H] exp(A_log)
    const float* f_bias;    // MODE_GATED: [H * d]
    const float* lower;     // MODE_GATED: [H * d]
    float* state;           // [slots][H][d][dv]
    long long state_stride;
    const int* q_start;
    const int* q_len;
    const int* slots;
    float* out;             // [T][H * dv]
    int H, G, d, dv, L;     // G heads of q and k (MODE_DELTA; head h reads h / (H / G))
};

template <int MODE>
__global__ __launch_bounds__(THREADS) void matrix_rnn_kernel(RnnArgs a) {
    extern __shared__ float sm[];
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.z, h = blockIdx.y;
    const int n = a.q_len[e];
    if (n <= 0) return;
    const int L = a.L, CT = THREADS / L, DP = L * R;
    const int d = a.d, dv = a.dv;
    float* q_s = sm;                    // [TB][DP]
    float* k_s = q_s + TB * DP;         // [TB][DP]   (MODE_GATED: the forget gate)
    float* v_s = k_s + TB * DP;         // [TB][CT]
    float* o_s = v_s + TB * CT;         // [TB][CT]
    float* g_s = o_s + TB * CT;         // [TB]
    float* b_s = g_s + TB;              // [TB]
    const int tid = threadIdx.x, kl = tid % L, col = tid / L;
    const int j = blockIdx.x * CT + col;
    const bool live = j < dv;
    const int lane = tid & 31, warp = tid >> 5;
    const int t0 = a.q_start[e];
    float* st = a.state + (size_t)a.slots[e] * a.state_stride + (size_t)h * d * dv;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = kl + L * r;
        S[r] = (live && i < d) ? st[(size_t)i * dv + j] : 0.f;
    }
    const int hk = MODE == MODE_DELTA ? h / (a.H / a.G) : h;
    const float qscale = rsqrtf((float)d);
    for (int b0 = 0; b0 < n; b0 += TB) {
        const int nb = min(TB, n - b0);
        __syncthreads();      // (everyone is done with the batch before)
        for (int idx = tid; idx < TB * DP; idx += THREADS) {
            const int tt = idx / DP, i = idx % DP;
            float q = 0.f, k = 0.f;
            if (tt < nb && i < d) {
                const long long t = t0 + b0 + tt;
                if (MODE == MODE_DELTA) {
                    q = a.x[t * a.ldx + a.q_col + hk * d + i];
                    k = a.x[t * a.ldx + a.k_col + hk * d + i];
                } else {
                    const int c = h * d + i;
                    q = silu_f(rows_at(a.u, t, a.q_col + c));
                    const float low = a.lower[c];
                    k = low + (1.f - low) * sigmoid_f(rows_at(a.u, t, a.k_col + c) + a.f_bias[c]);
                }
            }
            q_s[idx] = q;
            k_s[idx] = k;
        }
        for (int idx = tid; idx < TB * CT; idx += THREADS) {
            const int tt = idx / CT, c = blockIdx.x * CT + idx % CT;
            float v = 0.f;
            if (tt < nb && c < dv) {
                const long long t = t0 + b0 + tt;
                v = MODE == MODE_DELTA ? a.x[t * a.ldx + a.v_col + h * dv + c] : rows_at(a.u, t, a.v_col + h * dv + c);
            }
            v_s[idx] = v;
        }
        if (MODE == MODE_DELTA && tid < nb) {
            const long long t = t0 + b0 + tid;
            b_s[tid] = sigmoid_f(rows_at(a.u, t, a.b_col + h));
            g_s[tid] = expf(-a.rate[h] * softplus_f(rows_at(a.u, t, a.a_col + h) + a.dt_bias[h]));
        }
        __syncthreads();
        if (MODE == MODE_DELTA) {
            // q and k as unit vectors (a warp a token)
            for (int tt = warp; tt < nb; tt += THREADS / 32) {
                float sq = 0.f, sk = 0.f;
                for (int i = lane; i < d; i += 32) {
                    sq = fmaf(q_s[tt * DP + i], q_s[tt * DP + i], sq);
                    sk = fmaf(k_s[tt * DP + i], k_s[tt * DP + i], sk);
                }
                sq = warp_sum(sq);
                sk = warp_sum(sk);
                const float rq = rsqrtf(sq + 1e-6f) * qscale, rk = rsqrtf(sk + 1e-6f);
                for (int i = lane; i < d; i += 32) {
                    q_s[tt * DP + i] *= rq;
                    k_s[tt * DP + i] *= rk;
                }
            }
            __syncthreads();
        }
        for (int tt = 0; tt < nb; ++tt) {
            const float* qq = q_s + tt * DP + kl;
            const float* kk = k_s + tt * DP + kl;
            const float v = v_s[tt * CT + col];
            float o = 0.f;
            if (MODE == MODE_DELTA) {
                float p = 0.f;
#pragma unroll
                for (int r = 0; r < R; ++r) p = fmaf(S[r], kk[L * r], p);
                for (int off = 1; off < L; off <<= 1) p += __shfl_xor_sync(0xffffffffu, p, off);
                const float g = g_s[tt];
                const float w = b_s[tt] * (v - g * p);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    S[r] = fmaf(kk[L * r], w, g * S[r]);
                    o = fmaf(S[r], qq[L * r], o);
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float f = kk[L * r];
                    S[r] = fmaf(f, S[r], (1.f - f) * v);
                    o = fmaf(S[r], qq[L * r], o);
                }
            }
            for (int off = 1; off < L; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (kl == 0) o_s[tt * CT + col] = o;
        }
        __syncthreads();
        for (int idx = tid; idx < nb * CT; idx += THREADS) {
            const int tt = idx / CT, c = blockIdx.x * CT + idx % CT;
            if (c < dv) a.out[(size_t)(t0 + b0 + tt) * (a.H * dv) + h * dv + c] = o_s[tt * CT + idx % CT];
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = kl + L * r;
            if (i < d) st[(size_t)i * dv + j] = S[r];
        }
    }
}

// a warp a (token, head)
template <typename TOUT>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, Rows gate, int gate_col, const float* __restrict__ w, float eps,
                                      const int* __restrict__ q_start, const int* __restrict__ q_len, int E, int T, int H, int dv,
                                      TOUT* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)T * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const size_t base = (size_t)t * H * dv + (size_t)h * dv;
    if (entry_of_row(q_start, q_len, E, t) < 0) {
        for (int c = lane; c < dv; c += 32) out[base + c] = from_f32<TOUT>(0.f);
        return;
    }
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(o[base + c], o[base + c], ss);
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        float v = o[base + c] * rstd * w[c];
        if (gate.p != nullptr) v *= silu_f(rows_at(gate, t, gate_col + h * dv + c));
        out[base + c] = from_f32<TOUT>(v);
    }
}

int rnn_lanes(int d) {
    int L = 1;
    while (L * R < d) L <<= 1;
    return L;
}

}  // namespace

// mode 0: the gated delta rule; 1: the gated linear form (see the head of this file).  u [S][T][ld] the projection's sums;
// x [T][ldx] the convolved rows (mode 0).  state [slots][H][d][dv].  out [T][H * dv] 32-bit.  Entries of no tokens are left out.
VCB_API int vcb_matrix_rnn(int mode, const float* u, int S, long long s_stride, long long ld, const float* x, long long ldx,
                           int q_col, int k_col, int v_col, int b_col, int a_col, const float* dt_bias, const float* rate,
                           const float* f_bias, const float* lower, float* state, long long state_stride, const int* q_start,
                           const int* q_len, const int* slots, int E, int H, int G, int d, int dv, float* out,
                           cudaStream_t stream) {
    if (E == 0) return 0;
    VCB_CHECK_ARG(mode == 0 || mode == 1, "matrix_rnn: unknown mode %d", mode);
    VCB_CHECK_ARG(d >= 1 && d <= 32 * R, "matrix_rnn: %d state rows a head (1 to %d)", d, 32 * R);
    VCB_CHECK_ARG(H >= 1 && G >= 1 && H % G == 0 && dv >= 1, "matrix_rnn: bad sizes H=%d G=%d dv=%d", H, G, dv);
    VCB_CHECK_ARG(H <= 65535 && E <= 65535, "matrix_rnn: %d heads, %d entries", H, E);
    const int L = rnn_lanes(d), CT = THREADS / L, DP = L * R;
    RnnArgs a{Rows{u, S < 1 ? 1 : S, s_stride, ld}, x, ldx, q_col, k_col, v_col, b_col, a_col, dt_bias, rate, f_bias, lower, state,
              state_stride, q_start, q_len, slots, out, H, G, d, dv, L};
    const size_t smem = (size_t)(2 * TB * DP + 2 * TB * CT + 2 * TB) * sizeof(float);
    const dim3 grid((dv + CT - 1) / CT, H, E);
    if (mode == 0) launch_pdl(matrix_rnn_kernel<MODE_DELTA>, grid, dim3(THREADS), smem, stream, a);
    else launch_pdl(matrix_rnn_kernel<MODE_GATED>, grid, dim3(THREADS), smem, stream, a);
    VCB_CHECK_LAUNCH("matrix_rnn");
    return 0;
}

// o [T][H * dv] 32-bit; gate (or null) [S][T][ld] sums whose columns gate_col .. gate_col + H dv gate o through a SiLU; w [dv];
// out [T][H * dv] of out_dtype (zeros in rows outside every entry).
VCB_API int vcb_head_norm_gate(const float* o, const float* gate, int S, long long s_stride, long long ld, int gate_col,
                               const float* w, float eps, const int* q_start, const int* q_len, int E, int T, int H, int dv,
                               void* out, int out_dtype, cudaStream_t stream) {
    if (T == 0 || H == 0) return 0;
    const long long items = (long long)T * H;
    const int warps = 8;
    const dim3 grid((unsigned)((items + warps - 1) / warps));
    Rows g{gate, S < 1 ? 1 : S, s_stride, ld};
    if (out_dtype == VCB_F32)
        launch_pdl(head_norm_gate_kernel<float>, grid, dim3(32 * warps), 0, stream, o, g, gate_col, w, eps, q_start, q_len, E, T, H, dv, (float*)out);
    else
        launch_pdl(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(32 * warps), 0, stream, o, g, gate_col, w, eps, q_start, q_len, E, T, H,
                   dv, (__nv_bfloat16*)out);
    VCB_CHECK_LAUNCH("head_norm_gate");
    return 0;
}
