// Several residual streams instead of one ("hyper-connections"), and the token shift on what a mixer reads.
//
//  * hyper_mix_norm   one pass over a row of the S streams x_1 .. x_S (32-bit, [S][T][W]):
//                       write-back of the sublayer before:  x_r <- sum_s mix[s][r] x_s + out[r] * y      (all from the old ones)
//                       read-out for the sublayer ahead:    u = sum_r in[r] x_r
//                       its norm:                           h = gain * u / sqrt(mean(u^2) + eps)
//                     y arrives as 32-bit sums, possibly k-slice partial sums added here in slice order.  The first
//                     sublayer of a step has no write-back: its streams all start as the embedding's row (`init`).
//                     With a row list the streams are left as they are and only the listed rows are read out (the
//                     model's last norm on the rows whose logits are wanted; `in` null: the plain sum of the streams).
//                     h leaves in the compute dtype, or 32-bit where the token shift reads it next.
//  * token_shift      h_t <- h_t + (h_(t-1) - h_t) * mu per channel, h_(t-1) as it was before this replacement; the row
//                     before an entry's first comes from the request's state (zeros before its first token), which then
//                     takes the entry's last row.  The thread that reads a state element is the one that writes it.
//
// Everything is 32-bit arithmetic.  Rows of a captured step's padding are computed like any other (they are read by
// nothing); entries of no tokens touch no state.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

struct Rows {
    const float* p;       // [S][T][ld] 32-bit sums, or null
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

struct HyperArgs {
    float* streams;        // [S][T][W]
    const float* init;     // [T][W] or null: the streams all start as this row (nothing is read from `streams`)
    Rows y;                // the sublayer's result to write back (p null: none)
    const float* mix;      // [S][S], [from][to]
    const float* outw;     // [S]
    const float* inw;      // [S] or null: the plain sum
    const float* gain;     // [W] or null: no read-out at all
    float eps;
    void* out;             // [n][W] in out_dtype
    int out_dtype;
    const int* rows;       // or null
    int T, W, S;
};

template <typename TOUT>
__global__ void hyper_mix_norm_kernel(HyperArgs a) {
    extern __shared__ float u_s[];          // [W] the read-out of this row
    __shared__ float red[33];
    __shared__ float cm[MAX_STREAMS * MAX_STREAMS], co[MAX_STREAMS], ci[MAX_STREAMS];
    pdl_trigger();
    const int S = a.S, W = a.W;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) cm[i] = a.mix != nullptr ? a.mix[i] : (i / S == i % S ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        co[i] = a.outw != nullptr ? a.outw[i] : 1.f;
        ci[i] = a.inw != nullptr ? a.inw[i] : 1.f;
    }
    pdl_wait();
    __syncthreads();
    const int t = a.rows != nullptr ? a.rows[blockIdx.x] : blockIdx.x;
    const size_t plane = (size_t)a.T * W;
    float ss = 0.f;
    // rows of a multiple of four lanes on 16-byte boundaries move as 16-byte words (the same sums, lane by lane)
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = (W & 3) == 0 && aligned16(a.streams) && aligned16(a.init) && aligned16(a.gain) && aligned16(a.out) && aligned16(u_s) &&
                     aligned16(a.y.p) && (a.y.ld & 3) == 0 && (a.y.s_stride & 3) == 0;
    if (vec) {
        const int W4 = W >> 2;
        for (int c4 = threadIdx.x; c4 < W4; c4 += blockDim.x) {
            float4 x[MAX_STREAMS];
            if (a.init != nullptr) {
                const float4 v = reinterpret_cast<const float4*>(a.init + (size_t)t * W)[c4];
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s) x[s] = v;
            } else {
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s)
                    if (s < S) x[s] = reinterpret_cast<const float4*>(a.streams + s * plane + (size_t)t * W)[c4];
            }
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.y.p != nullptr) {
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                const float* yp = a.y.p + (long long)t * a.y.ld;
                for (int k = 0; k < a.y.S; ++k) {
                    const float4 part = reinterpret_cast<const float4*>(yp + (long long)k * a.y.s_stride)[c4];
                    y.x += part.x; y.y += part.y; y.z += part.z; y.w += part.w;
                }
#pragma unroll
                for (int r = 0; r < MAX_STREAMS; ++r) {
                    if (r < S) {
                        float4 n = make_float4(co[r] * y.x, co[r] * y.y, co[r] * y.z, co[r] * y.w);
#pragma unroll
                        for (int s2 = 0; s2 < MAX_STREAMS; ++s2)
                            if (s2 < S) {
                                const float m = cm[s2 * S + r];
                                n.x = fmaf(m, x[s2].x, n.x); n.y = fmaf(m, x[s2].y, n.y); n.z = fmaf(m, x[s2].z, n.z); n.w = fmaf(m, x[s2].w, n.w);
                            }
                        if (a.rows == nullptr) reinterpret_cast<float4*>(a.streams + r * plane + (size_t)t * W)[c4] = n;
                        u.x = fmaf(ci[r], n.x, u.x); u.y = fmaf(ci[r], n.y, u.y); u.z = fmaf(ci[r], n.z, u.z); u.w = fmaf(ci[r], n.w, u.w);
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < MAX_STREAMS; ++r) {
                    if (r < S) {
                        if (a.init != nullptr && a.rows == nullptr) reinterpret_cast<float4*>(a.streams + r * plane + (size_t)t * W)[c4] = x[r];
                        u.x = fmaf(ci[r], x[r].x, u.x); u.y = fmaf(ci[r], x[r].y, u.y); u.z = fmaf(ci[r], x[r].z, u.z); u.w = fmaf(ci[r], x[r].w, u.w);
                    }
                }
            }
            reinterpret_cast<float4*>(u_s)[c4] = u;
            ss = fmaf(u.w, u.w, fmaf(u.z, u.z, fmaf(u.y, u.y, fmaf(u.x, u.x, ss))));
        }
        if (a.gain == nullptr) return;
        ss = block_sum(ss, red);
        const float rstd = rsqrtf(ss / (float)W + a.eps);
        TOUT* o = (TOUT*)a.out + (size_t)blockIdx.x * W;
        for (int c4 = threadIdx.x; c4 < W4; c4 += blockDim.x) {
            const float4 u = reinterpret_cast<const float4*>(u_s)[c4], g = reinterpret_cast<const float4*>(a.gain)[c4];
            o[4 * c4] = from_f32<TOUT>(u.x * rstd * g.x);
            o[4 * c4 + 1] = from_f32<TOUT>(u.y * rstd * g.y);
            o[4 * c4 + 2] = from_f32<TOUT>(u.z * rstd * g.z);
            o[4 * c4 + 3] = from_f32<TOUT>(u.w * rstd * g.w);
        }
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[MAX_STREAMS];
        if (a.init != nullptr) {
            const float v = a.init[(size_t)t * W + c];
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s) x[s] = v;
        } else {
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) x[s] = a.streams[s * plane + (size_t)t * W + c];
        }
        float u = 0.f;
        if (a.y.p != nullptr) {
            const float y = rows_at(a.y, t, c);
#pragma unroll
            for (int r = 0; r < MAX_STREAMS; ++r) {
                if (r < S) {
                    float n = co[r] * y;
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s)
                        if (s < S) n = fmaf(cm[s * S + r], x[s], n);
                    if (a.rows == nullptr) a.streams[r * plane + (size_t)t * W + c] = n;
                    u = fmaf(ci[r], n, u);
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < MAX_STREAMS; ++r) {
                if (r < S) {
                    if (a.init != nullptr && a.rows == nullptr) a.streams[r * plane + (size_t)t * W + c] = x[r];
                    u = fmaf(ci[r], x[r], u);
                }
            }
        }
        u_s[c] = u;
        ss = fmaf(u, u, ss);
    }
    if (a.gain == nullptr) return;
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)W + a.eps);
    TOUT* o = (TOUT*)a.out + (size_t)blockIdx.x * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) o[c] = from_f32<TOUT>(u_s[c] * rstd * a.gain[c]);
}

template <typename TOUT>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                                   long long state_stride, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ slots, int E, int T, int W, TOUT* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const int e = entry_of_row(q_start, q_len, E, t);
        if (e < 0) continue;
        const int first = q_start[e], n = q_len[e];
        float* st = state + (size_t)slots[e] * state_stride;
        for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < W; c += gridDim.x * blockDim.x) {
            const float v = h[(size_t)t * W + c];
            float prev;
            if (t == first) {
                prev = st[c];
                st[c] = h[(size_t)(first + n - 1) * W + c];
            } else {
                prev = h[(size_t)(t - 1) * W + c];
            }
            out[(size_t)t * W + c] = from_f32<TOUT>(fmaf(prev - v, mu[c], v));
        }
    }
}

}  // namespace

// streams [S][T][W] 32-bit.  init (or null) [T][W]: the step's first sublayer, every stream starts as this row.  y (or null)
// [Sy][T][ldy]: the result of the sublayer before, written back through mix [S][S] ([from][to]) and outw [S] (null: the
// identity and ones).  inw [S] (null: ones), gain [W], eps: the read-out and its norm into out [n][W] of out_dtype (gain
// null: no read-out).  rows (or null): n_rows row indices, the streams are then only read.
VCB_API int vcb_hyper_mix_norm(float* streams, const float* init, const float* y, int Sy, long long y_stride, long long ldy,
                               const float* mix, const float* outw, const float* inw, const float* gain, float eps, void* out,
                               int out_dtype, const int* rows, int n_rows, int T, int W, int S, cudaStream_t stream) {
    const int n = rows != nullptr ? n_rows : T;
    if (n == 0) return 0;
    VCB_CHECK_ARG(S >= 1 && S <= MAX_STREAMS, "hyper_mix_norm: %d streams (1 to %d)", S, MAX_STREAMS);
    VCB_CHECK_ARG((gain == nullptr) == (out == nullptr), "hyper_mix_norm: a read-out needs both its gain and its output");
    const size_t smem = (size_t)W * sizeof(float);
    VCB_CHECK_ARG(smem <= 200 * 1024, "hyper_mix_norm: a width of %d is more than the kernel's shared memory holds", W);
    HyperArgs a{streams, init, Rows{y, Sy < 1 ? 1 : Sy, y_stride, ldy}, mix, outw, inw, gain, eps, out, out_dtype, rows, T, W, S};
    const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
    if (out_dtype == VCB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_mix_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(hyper_mix_norm_kernel<float>, dim3(n), dim3(threads), smem, stream, a);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_mix_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(hyper_mix_norm_kernel<__nv_bfloat16>, dim3(n), dim3(threads), smem, stream, a);
    }
    VCB_CHECK_LAUNCH("hyper_mix_norm");
    return 0;
}

// h [T][W] 32-bit; mu [W]; state [slots][state_stride]: the last row every request's mixer input had; out [T][W].
VCB_API int vcb_token_shift(const float* h, const float* mu, float* state, long long state_stride, const int* q_start,
                            const int* q_len, const int* slots, int E, int T, int W, void* out, int out_dtype,
                            cudaStream_t stream) {
    if (T == 0 || E == 0) return 0;
    const dim3 grid((W + 255) / 256, T < 65535 ? T : 65535);
    if (out_dtype == VCB_F32)
        launch_pdl(token_shift_kernel<float>, grid, dim3(256), 0, stream, h, mu, state, state_stride, q_start, q_len, slots, E, T, W, (float*)out);
    else
        launch_pdl(token_shift_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, h, mu, state, state_stride, q_start, q_len, slots, E, T,
                   W, (__nv_bfloat16*)out);
    VCB_CHECK_LAUNCH("token_shift");
    return 0;
}
