// A feed-forward made of many small experts, of which a router picks a few per token:
//
//  * moe_route     per token: the router's logits (32-bit sums) -> the `top` experts with the largest logits and their
//                  weights (the sigmoid or, over the chosen ones, the softmax of the logits)
//  * moe_group     the step's (token, choice) pairs sorted by expert: every expert's pairs fill whole tiles of BM rows
//                  (the last one padded), so that a tile of rows meets the weights of one expert only
//  * moe_gemm      the experts' products over those tiles: the up projection reads the tokens' rows through the sorted
//                  order (times the pair's weight where the weight belongs on the expert's input, rounded to the
//                  compute dtype as a stored activation would be) and applies the activation; the down projection
//                  writes 32-bit sums per pair
//  * moe_combine   per token: the sums of its pairs, in the order the router chose them (times the pair's weight where
//                  it belongs on the output), plus a shared expert's result
//
// Nothing here asks the host how many tokens an expert got: the grids are laid out for the most tiles the step can
// need and a tile beyond the last one returns at once, so a captured step replays it.  Products accumulate in 32-bit
// in a fixed order over the inner dimension, whatever tile a row lands in.
#include "common.cuh"

#include <math_constants.h>

namespace {

constexpr int BM = 32;    // rows (pairs) per tile of the plain product below
constexpr int BN = 64;    // output features per block
constexpr int BK = 16;

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

// a warp a token; the logits of the warp's token lie in shared memory while its lanes look for the next largest
__global__ void moe_route_kernel(Rows logits, const int* __restrict__ q_start, const int* __restrict__ q_len, int n_entries,
                                 int T, int E, int top, int softmax_weights, int* __restrict__ sel_e, float* __restrict__ sel_w) {
    extern __shared__ float zs[];   // [warps][E]
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    if (entry_of_row(q_start, q_len, n_entries, t) < 0) {
        for (int k = lane; k < top; k += 32) sel_e[(size_t)t * top + k] = -1;
        return;
    }
    float* z = zs + (size_t)warp * E;
    for (int e = lane; e < E; e += 32) z[e] = rows_at(logits, t, e);
    __syncwarp();
    float first = 0.f, denom = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -CUDART_INF_F;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at && v != -CUDART_INF_F)) { best = v; at = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (k == 0) first = best;
        if (lane == 0) {
            sel_e[(size_t)t * top + k] = at;
            // sigmoid of the logit as it is, or (softmax over the chosen) exp(z - z_first), divided below
            sel_w[(size_t)t * top + k] = softmax_weights ? expf(best - first) : 1.f / (1.f + expf(-best));
            z[at] = -CUDART_INF_F;
        }
        denom += expf(best - first);
        __syncwarp();
    }
    if (softmax_weights)
        for (int k = lane; k < top; k += 32) sel_w[(size_t)t * top + k] /= denom;
}

// The same for routers that choose by a corrected score among the experts of the best groups: s = sigmoid(z); the choice
// score is s + correction; the E experts form `n_groups` equal groups of neighbours, a group's score is the sum of its
// two largest choice scores, and only experts of the `keep` best groups can be chosen (the others count as minus
// infinity, so a negative choice score inside a kept group still beats them); the `top` largest choice scores win
// (the lowest index on a tie); a chosen expert's weight is s * weight_scale, without the correction, not renormalised.
__global__ void moe_route_grouped_kernel(Rows logits, const float* __restrict__ correction, int n_groups, int keep,
                                         float weight_scale, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                         int n_entries, int T, int E, int top, int* __restrict__ sel_e,
                                         float* __restrict__ sel_w) {
    extern __shared__ float zs[];   // [warps][2 E + n_groups]
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    if (entry_of_row(q_start, q_len, n_entries, t) < 0) {
        for (int k = lane; k < top; k += 32) sel_e[(size_t)t * top + k] = -1;
        return;
    }
    float* s = zs + (size_t)warp * (2 * E + n_groups);
    float* c = s + E;
    float* gs = c + E;
    for (int e = lane; e < E; e += 32) {
        const float v = 1.f / (1.f + expf(-rows_at(logits, t, e)));
        s[e] = v;
        c[e] = v + (correction != nullptr ? correction[e] : 0.f);
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -CUDART_INF_F, b = -CUDART_INF_F;     // the two largest
            for (int i = 0; i < per; ++i) {
                const float v = c[g * per + i];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the `keep` best groups are marked by NaN-free flags: a kept group's score becomes +inf
        for (int k = 0; k < keep; ++k) {
            float best = -CUDART_INF_F;
            int at = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v != CUDART_INF_F && (v > best || (v == best && g < at))) { best = v; at = g; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
            }
            if (lane == 0 && at != 0x7fffffff) gs[at] = CUDART_INF_F;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != CUDART_INF_F) c[e] = -CUDART_INF_F;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -CUDART_INF_F;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (v != -CUDART_INF_F && (v > best || (v == best && e < at))) { best = v; at = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
        }
        if (lane == 0) {
            // (fewer allowed experts than `top` cannot happen for a well-formed router; the choice then names none)
            sel_e[(size_t)t * top + k] = at == 0x7fffffff ? -1 : at;
            sel_w[(size_t)t * top + k] = at == 0x7fffffff ? 0.f : s[at] * weight_scale;
            if (at != 0x7fffffff) c[at] = -CUDART_INF_F;
        }
        __syncwarp();
    }
}

// one block: counts, padded offsets, the tiles' experts, then every pair's place
__global__ void moe_group_kernel(const int* __restrict__ sel_e, int A, int E, int tiles_cap, int BM, int* __restrict__ pos_of,
                                 int* __restrict__ src_of, int* __restrict__ tile_expert) {
    extern __shared__ int sh[];    // cnt[E], off[E]
    pdl_trigger();
    pdl_wait();
    int* cnt = sh;
    int* off = sh + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = sel_e[a];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    for (int i = threadIdx.x; i < tiles_cap * BM; i += blockDim.x) src_of[i] = -1;
    for (int i = threadIdx.x; i < tiles_cap; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = tile * BM;
            const int n = (cnt[e] + BM - 1) / BM;
            for (int i = 0; i < n && tile < tiles_cap; ++i) tile_expert[tile++] = e;
            cnt[e] = 0;
        }
    }
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = sel_e[a];
        int pos = -1;
        if (e >= 0 && e < E) {
            pos = off[e] + atomicAdd(&cnt[e], 1);
            if (pos < tiles_cap * BM) src_of[pos] = a;
            else pos = -1;
        }
        pos_of[a] = pos;
    }
}

struct GemmArgs {
    const void* x;        // GATHER: the tokens' rows [T][ldx]; else the pairs' rows in sorted order [rows][ldx]
    long long ldx;
    const void* w;        // [E][N][K]
    const int* tile_expert;
    const int* src_of;    // GATHER: sorted place -> pair (token * top + choice), -1: padding
    const float* sel_w;   // GATHER: the pairs' weights, or null: rows are read as they are
    int top;
    void* out;            // [rows][N]: the compute dtype with an activation, else 32-bit
    int N, K;
    int act;              // -1: none (32-bit out); else the activation's number
};

__device__ __forceinline__ float act_of(float x, int kind) {
    switch (kind) {
        case 0: return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
        case 1: return 0.5f * x * (1.f + tanhf(0.79788456080286535588f * (x + 0.044715f * x * x * x)));
        case 2: return x / (1.f + expf(-x));
        case 3: { const float r = fmaxf(x, 0.f); return r * r; }
        default: return x;
    }
}

// grid (tiles, ceil(N / BN)); 256 threads, two rows by four features each; k runs in order
template <typename T, bool GATHER>
__global__ __launch_bounds__(256) void moe_gemm_kernel(GemmArgs a) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int src_s[BM];
    __shared__ float wt_s[BM];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    const int e = a.tile_expert[tile];
    if (e < 0) return;
    const int tid = threadIdx.x;
    const int n0 = blockIdx.y * BN;
    if (tid < BM) {
        int src = tile * BM + tid;
        float wt = 1.f;
        if (GATHER) {
            const int pair = a.src_of[src];
            src = pair < 0 ? -1 : pair / a.top;
            if (pair >= 0 && a.sel_w != nullptr) wt = a.sel_w[pair];
        }
        src_s[tid] = src;
        wt_s[tid] = wt;
    }
    __syncthreads();
    const T* x = reinterpret_cast<const T*>(a.x);
    const T* w = reinterpret_cast<const T*>(a.w) + (size_t)e * a.N * a.K;
    const int ty = tid >> 4, tx = tid & 15;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < a.K; k0 += BK) {
        for (int i = tid; i < BM * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            const int src = src_s[r];
            float v = 0.f;
            if (src >= 0 && k0 + k < a.K) {
                v = to_f32(x[(size_t)src * a.ldx + k0 + k]);
                if (GATHER && a.sel_w != nullptr) v = to_f32(from_f32<T>(v * wt_s[r]));
            }
            As[k][r] = v;
        }
        for (int i = tid; i < BN * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            Ws[k][r] = (n0 + r < a.N && k0 + k < a.K) ? to_f32(w[(size_t)(n0 + r) * a.K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float a0 = As[k][2 * ty], a1 = As[k][2 * ty + 1];
            const float4 b = *reinterpret_cast<const float4*>(&Ws[k][4 * tx]);
            acc[0][0] = fmaf(a0, b.x, acc[0][0]); acc[0][1] = fmaf(a0, b.y, acc[0][1]);
            acc[0][2] = fmaf(a0, b.z, acc[0][2]); acc[0][3] = fmaf(a0, b.w, acc[0][3]);
            acc[1][0] = fmaf(a1, b.x, acc[1][0]); acc[1][1] = fmaf(a1, b.y, acc[1][1]);
            acc[1][2] = fmaf(a1, b.z, acc[1][2]); acc[1][3] = fmaf(a1, b.w, acc[1][3]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const size_t row = (size_t)tile * BM + 2 * ty + i;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + 4 * tx + j;
            if (n < a.N) {
                if (a.act >= 0) reinterpret_cast<T*>(a.out)[row * a.N + n] = from_f32<T>(act_of(acc[i][j], a.act));
                else reinterpret_cast<float*>(a.out)[row * a.N + n] = acc[i][j];
            }
        }
    }
}

// a block a sorted row: the token's row times the pair's weight, rounded to the compute dtype (zeros in padding rows)
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ src_of,
                                  const float* __restrict__ sel_w, int top, int K, T* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int pos = blockIdx.x;
    const int pair = src_of[pos];
    T* dst = out + (size_t)pos * K;
    if (pair < 0) {
        for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = from_f32<T>(0.f);
        return;
    }
    const T* src = x + (size_t)(pair / top) * ldx;
    const float w = sel_w != nullptr ? sel_w[pair] : 1.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = from_f32<T>(to_f32(src[k]) * w);
}

// grid (ceil(W / 256), rows): out[t] = shared[t] + sum over the token's pairs, in the router's order
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of, const float* __restrict__ sel_w,
                                   int top, Rows shared, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   int n_entries, int W, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W || entry_of_row(q_start, q_len, n_entries, t) < 0) return;
    float v = shared.p != nullptr ? rows_at(shared, t, c) : 0.f;
    for (int k = 0; k < top; ++k) {
        const int pos = pos_of[(size_t)t * top + k];
        if (pos >= 0) {
            const float r = y[(size_t)pos * W + c];
            v += sel_w != nullptr ? r * sel_w[(size_t)t * top + k] : r;
        }
    }
    out[(size_t)t * W + c] = v;
}

// four channels a thread (W a multiple of 4, every base and stride a multiple of 4 elements)
__global__ void moe_combine_vec_kernel(const float* __restrict__ y, const int* __restrict__ pos_of, const float* __restrict__ sel_w,
                                       int top, Rows shared, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                       int n_entries, int W, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (c >= W || entry_of_row(q_start, q_len, n_entries, t) < 0) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shared.p != nullptr) {
        const float* p = shared.p + (long long)t * shared.ld + c;
        for (int s = 0; s < shared.S; ++s) {
            const float4 a = *reinterpret_cast<const float4*>(p + (long long)s * shared.s_stride);
            v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
        }
    }
    for (int k = 0; k < top; ++k) {
        const int pos = pos_of[(size_t)t * top + k];
        if (pos >= 0) {
            const float4 r = *reinterpret_cast<const float4*>(y + (size_t)pos * W + c);
            const float wt = sel_w != nullptr ? sel_w[(size_t)t * top + k] : 1.f;
            if (sel_w != nullptr) { v.x += r.x * wt; v.y += r.y * wt; v.z += r.z * wt; v.w += r.w * wt; }
            else { v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; }
        }
    }
    *reinterpret_cast<float4*>(out + (size_t)t * W + c) = v;
}

}  // namespace

VCB_API int vcb_moe_tile_rows() { return BM; }

// logits [S][T][ld] 32-bit sums with E columns.  sel_e, sel_w [T * top]: expert (-1 for rows outside every entry) and weight of
// each choice.  softmax_weights 0: the sigmoid of the chosen logit; 1: the softmax over the chosen logits.
VCB_API int vcb_moe_route(const float* logits, int S, long long s_stride, long long ld, const int* q_start, const int* q_len,
                          int n_entries, int T, int E, int top, int softmax_weights, int* sel_e, float* sel_w,
                          cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(E >= 1 && top >= 1 && top <= E, "moe_route: %d of %d experts", top, E);
    const int warps = 4;
    const size_t smem = (size_t)warps * E * sizeof(float);
    VCB_CHECK_ARG(smem <= 48 * 1024, "moe_route: %d experts are more than the kernel's shared memory holds", E);
    launch_pdl(moe_route_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), smem, stream,
               Rows{logits, S < 1 ? 1 : S, s_stride, ld}, q_start, q_len, n_entries, T, E, top, softmax_weights, sel_e, sel_w);
    VCB_CHECK_LAUNCH("moe_route");
    return 0;
}

// The router of grouped experts with a corrected choice score (see moe_route_grouped_kernel).  correction [E] or null;
// n_groups divides E; keep of them can be chosen from (n_groups <= 1 or keep >= n_groups: all experts are open).
VCB_API int vcb_moe_route_grouped(const float* logits, int S, long long s_stride, long long ld, const float* correction,
                                  int n_groups, int keep, float weight_scale, const int* q_start, const int* q_len,
                                  int n_entries, int T, int E, int top, int* sel_e, float* sel_w, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(E >= 1 && top >= 1 && top <= E, "moe_route_grouped: %d of %d experts", top, E);
    if (n_groups < 1) n_groups = 1;
    VCB_CHECK_ARG(E % n_groups == 0, "moe_route_grouped: %d experts in %d equal groups", E, n_groups);
    VCB_CHECK_ARG(n_groups == 1 || keep >= 1, "moe_route_grouped: %d groups kept", keep);
    VCB_CHECK_ARG(n_groups == 1 || keep >= n_groups || (long long)keep * (E / n_groups) >= top,
                  "moe_route_grouped: %d groups of %d experts cannot give %d choices", keep, E / n_groups, top);
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + n_groups) * sizeof(float);
    VCB_CHECK_ARG(smem <= 48 * 1024, "moe_route_grouped: %d experts are more than the kernel's shared memory holds", E);
    launch_pdl(moe_route_grouped_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), smem, stream,
               Rows{logits, S < 1 ? 1 : S, s_stride, ld}, correction, n_groups, keep, weight_scale, q_start, q_len, n_entries, T, E,
               top, sel_e, sel_w);
    VCB_CHECK_LAUNCH("moe_route_grouped");
    return 0;
}

// A = T * top pairs, tiles of tile_rows rows.  pos_of [A]: a pair's row in the sorted order (-1: none); src_of [tiles_cap * tile_rows]: the pair in a row
// (-1: padding); tile_expert [tiles_cap]: the expert of a tile (-1: beyond the last).
VCB_API int vcb_moe_group(const int* sel_e, int A, int E, int tiles_cap, int tile_rows, int* pos_of, int* src_of,
                          int* tile_expert, cudaStream_t stream) {
    if (A == 0) return 0;
    VCB_CHECK_ARG(tile_rows >= 1, "moe_group: tiles of %d rows", tile_rows);
    const size_t smem = (size_t)2 * E * sizeof(int);
    VCB_CHECK_ARG(smem <= 48 * 1024, "moe_group: %d experts are more than the kernel's shared memory holds", E);
    launch_pdl(moe_group_kernel, dim3(1), dim3(1024), smem, stream, sel_e, A, E, tiles_cap, tile_rows, pos_of, src_of, tile_expert);
    VCB_CHECK_LAUNCH("moe_group");
    return 0;
}

// The experts' product over the sorted tiles.  w [E][N][K] of `dtype`.  gather != 0: x is the tokens' rows [T][ldx], read
// through src_of and multiplied by sel_w (null: not multiplied); else x is [tiles_cap * BM][ldx] in sorted order.
// act >= 0: out [tiles_cap * BM][N] of `dtype` after that activation; act < 0: out 32-bit sums.
VCB_API int vcb_moe_gemm(const void* x, long long ldx, const void* w, int dtype, const int* tile_expert, const int* src_of,
                         const float* sel_w, int top, int gather, void* out, int N, int K, int act, int tiles_cap,
                         cudaStream_t stream) {
    if (tiles_cap == 0) return 0;
    VCB_CHECK_ARG(act <= 3, "moe_gemm: unknown activation %d", act);
    VCB_CHECK_ARG(!gather || src_of != nullptr, "moe_gemm: gathering rows needs the sorted order");
    GemmArgs a{x, ldx, w, tile_expert, src_of, sel_w, top, out, N, K, act};
    const dim3 grid(tiles_cap, (N + BN - 1) / BN);
    if (dtype == VCB_F32) {
        if (gather) launch_pdl(moe_gemm_kernel<float, true>, grid, dim3(256), 0, stream, a);
        else launch_pdl(moe_gemm_kernel<float, false>, grid, dim3(256), 0, stream, a);
    } else {
        if (gather) launch_pdl(moe_gemm_kernel<__nv_bfloat16, true>, grid, dim3(256), 0, stream, a);
        else launch_pdl(moe_gemm_kernel<__nv_bfloat16, false>, grid, dim3(256), 0, stream, a);
    }
    VCB_CHECK_LAUNCH("moe_gemm");
    return 0;
}

// The tokens' rows in sorted order for a product that cannot read them through the order itself: out[pos] = x[token of
// the pair at pos] * sel_w[pair] (null: as it is), zeros where no pair sits.  x [T][ldx], out [rows][K], both `dtype`.
VCB_API int vcb_moe_gather(const void* x, long long ldx, int dtype, const int* src_of, const float* sel_w, int top, int rows,
                           int K, void* out, cudaStream_t stream) {
    if (rows == 0) return 0;
    const int threads = K >= 2048 ? 256 : 128;
    if (dtype == VCB_F32)
        launch_pdl(moe_gather_kernel<float>, dim3(rows), dim3(threads), 0, stream, (const float*)x, ldx, src_of, sel_w, top, K, (float*)out);
    else
        launch_pdl(moe_gather_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, (const __nv_bfloat16*)x, ldx, src_of, sel_w, top, K,
                   (__nv_bfloat16*)out);
    VCB_CHECK_LAUNCH("moe_gather");
    return 0;
}

// y [tiles_cap * BM][W] 32-bit sums per pair; shared (or null): a shared expert's sums [S][T][ld]; sel_w (or null): the
// pairs' weights where they belong on the output; out [T][W] 32-bit.
VCB_API int vcb_moe_combine(const float* y, const int* pos_of, const float* sel_w, int top, const float* shared, int S,
                            long long s_stride, long long ld, const int* q_start, const int* q_len, int n_entries, int T, int W,
                            float* out, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(T <= 65535, "moe_combine: %d rows in one step (at most 65535)", T);
    if (W % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0 &&
        (shared == nullptr || ((uintptr_t)shared % 16 == 0 && ld % 4 == 0 && (S <= 1 || s_stride % 4 == 0)))) {
        launch_pdl(moe_combine_vec_kernel, dim3((W / 4 + 127) / 128, T), dim3(128), 0, stream, y, pos_of, sel_w, top,
                   Rows{shared, S < 1 ? 1 : S, s_stride, ld}, q_start, q_len, n_entries, W, out);
        VCB_CHECK_LAUNCH("moe_combine");
        return 0;
    }
    launch_pdl(moe_combine_kernel, dim3((W + 255) / 256, T), dim3(256), 0, stream, y, pos_of, sel_w, top,
               Rows{shared, S < 1 ? 1 : S, s_stride, ld}, q_start, q_len, n_entries, W, out);
    VCB_CHECK_LAUNCH("moe_combine");
    return 0;
}
