// Attention whose keys and values are read out of one small latent vector per token.
//
// Per token the cache holds c (the normed latent, `kv_rank` lanes) and one rotated key part shared by all heads
// (`rot` lanes).  Head h's key is [W_uk[h] c | k_rot] and its value W_uv[h] c, so
//     q_h . k_h = (W_uk[h]^T q_h,plain) . c + q_h,rot . k_rot        and        sum_j w_j v_j = W_uv[h] (sum_j w_j c_j):
// with the queries carried into the latent space first, attention runs over the latent rows themselves as one shared
// KV head of kv_rank + rot key lanes whose values are the first kv_rank of them, and the heads' values are expanded
// afterwards.  The kernels here are the steps around that attention:
//
//  * latent_norm_rope_store   from the stacked down projections [q latent | kv latent | rotated key part] (32-bit sums):
//                             c_q = g_q n(q latent) to a buffer; c = g_kv n(kv latent) and the rotated key part to the
//                             token's cache row (key row [c | k_rot], value row c)
//  * head_linear              out[t, h, :] = M[h] in[t, h, :] for every head's own small matrix (queries into the latent
//                             space, latent sums out to the heads' values)
//  * rope_rows                the rotation alone, on a slice of every head of a 32-bit buffer (the queries' rotated part)
//
// Rotation pairs lane i with lane i + dims / 2; the angle is position * freq[i] in 32-bit, cos and sin times `gain`.
// Norms, angles and all sums are 32-bit.
#include "common.cuh"

namespace {

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

struct LatentArgs {
    Rows u;                 // [T][q_rank + kv_rank + rot]
    const float* gq;        // [q_rank]
    const float* gkv;       // [kv_rank]
    float eps;
    const int* positions;
    const float* freq;      // [rot / 2]
    float gain;
    const int* slot_map;    // token -> page * page_size + offset, -1: stored nowhere
    void* cq_out;           // [T][q_rank]
    void* pages;
    long long page_stride;
    int page_size, num_pages;
    int q_rank, kv_rank, rot, T;
    int v_width;            // lanes of a value row: kv_rank, or more (the lanes behind the latent are zeros)
    int* status;
};

template <typename TC>
__global__ void latent_norm_rope_store_kernel(LatentArgs a) {
    extern __shared__ float row[];          // [q_rank + kv_rank + rot]
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int nq = a.q_rank, nk = a.kv_rank, nr = a.rot, n = nq + nk + nr;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = rows_at(a.u, t, c);
        row[c] = v;
        if (c < nq) sq = fmaf(v, v, sq);
        else if (c < nq + nk) sk = fmaf(v, v, sk);
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float rq = rsqrtf(sq / (float)nq + a.eps), rk = rsqrtf(sk / (float)nk + a.eps);
    TC* cq = (TC*)a.cq_out + (size_t)t * nq;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) cq[c] = from_f32<TC>(row[c] * rq * a.gq[c]);
    const int slot = a.slot_map[t];
    if (slot < 0) return;
    const int page = slot / a.page_size, off = slot % a.page_size;
    if (page >= a.num_pages) {
        if (threadIdx.x == 0) atomicOr(a.status, VCB_STATUS_BAD_PAGE);
        return;
    }
    const int hd = nk + nr;
    TC* base = (TC*)a.pages + (size_t)page * a.page_stride;
    TC* krow = base + (size_t)off * hd;
    TC* vrow = base + (size_t)a.page_size * hd + (size_t)off * a.v_width;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const TC v = from_f32<TC>(row[nq + c] * rk * a.gkv[c]);
        krow[c] = v;
        vrow[c] = v;
    }
    for (int c = nk + threadIdx.x; c < a.v_width; c += blockDim.x) vrow[c] = from_f32<TC>(0.f);
    const int half = nr / 2;
    const float pos = (float)a.positions[t];
    const float* r = row + nq + nk;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * a.freq[i], &sn, &cs);
        sn *= a.gain;
        cs *= a.gain;
        const float x = r[i], y = r[i + half];
        krow[nk + i] = from_f32<TC>(x * cs - y * sn);
        krow[nk + half + i] = from_f32<TC>(y * cs + x * sn);
    }
    for (int i = 2 * half + threadIdx.x; i < nr; i += blockDim.x) krow[nk + i] = from_f32<TC>(r[i]);
}

// One block: head h, a tile of TT tokens.  A warp an output lane: its lanes walk the inner dimension (coalesced reads of the
// matrix row), every token of the tile takes its sum from the same pass over that row.
constexpr int HL_TOKENS = 8;

struct HeadLinearArgs {
    const void* in;         // [S][T][ld_in]: 32-bit sums (in_dtype F32) or one buffer of the compute dtype
    int in_dtype;
    int S;
    long long s_stride, ld_in;
    int in_head_stride, in_off;     // head h reads lanes [h * in_head_stride + in_off, + n_in)
    const void* m;          // [H][n_out][n_in] in m_dtype
    int m_dtype;
    void* out;              // [T][ld_out] in out_dtype; head h writes lanes [h * out_head_stride + out_off, + n_out)
    int out_dtype;
    long long ld_out;
    int out_head_stride, out_off;
    int T, H, n_in, n_out;
};

__global__ void head_linear_kernel(HeadLinearArgs a) {
    extern __shared__ float x_s[];          // [HL_TOKENS][n_in]
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.y, t0 = blockIdx.x * HL_TOKENS;
    const int nt = min(HL_TOKENS, a.T - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < HL_TOKENS * a.n_in; i += blockDim.x) {
        const int tt = i / a.n_in, c = i % a.n_in;
        float v = 0.f;
        if (tt < nt) {
            const size_t at = (size_t)(t0 + tt) * a.ld_in + (size_t)h * a.in_head_stride + a.in_off + c;
            if (a.in_dtype == VCB_F32) {
                for (int s = 0; s < a.S; ++s) v += ((const float*)a.in)[at + (size_t)s * a.s_stride];
            } else {
                v = __bfloat162float(((const __nv_bfloat16*)a.in)[at]);
            }
        }
        x_s[i] = v;
    }
    __syncthreads();
    for (int j = warp; j < a.n_out; j += nwarps) {
        float acc[HL_TOKENS];
#pragma unroll
        for (int tt = 0; tt < HL_TOKENS; ++tt) acc[tt] = 0.f;
        const size_t mrow = ((size_t)h * a.n_out + j) * a.n_in;
        for (int c = lane; c < a.n_in; c += 32) {
            const float w = load_as_f32(a.m, a.m_dtype, mrow + c);
#pragma unroll
            for (int tt = 0; tt < HL_TOKENS; ++tt) acc[tt] = fmaf(w, x_s[tt * a.n_in + c], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < HL_TOKENS; ++tt) acc[tt] = warp_sum(acc[tt]);
        if (lane < nt) {
            float v = acc[0];
#pragma unroll
            for (int tt = 1; tt < HL_TOKENS; ++tt)
                if (lane == tt) v = acc[tt];
            store_from_f32(a.out, a.out_dtype, (size_t)(t0 + lane) * a.ld_out + (size_t)h * a.out_head_stride + a.out_off + j, v);
        }
    }
}

struct RopeArgs {
    Rows in;                // [T][...]: head h's slice starts at lane h * in_head_stride + in_off
    int in_head_stride, in_off;
    const int* positions;
    const float* freq;      // [dims / 2]
    float gain;
    void* out;
    int out_dtype;
    long long ld_out;
    int out_head_stride, out_off;
    int T, H, dims, width;  // `width` lanes of the slice are copied, the first `dims` of them rotated
};

__global__ void rope_rows_kernel(RopeArgs a) {
    pdl_trigger();
    pdl_wait();
    const int half = a.dims / 2;
    const int per_head = half + (a.width - 2 * half);     // one thread a pair, one a lane that passes unchanged
    for (int t = blockIdx.y; t < a.T; t += gridDim.y) {
        const float pos = (float)a.positions[t];
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < a.H * per_head; i += gridDim.x * blockDim.x) {
            const int h = i / per_head, k = i % per_head;
            const int ib = h * a.in_head_stride + a.in_off;
            const size_t ob = (size_t)t * a.ld_out + (size_t)h * a.out_head_stride + a.out_off;
            if (k < half) {
                float sn, cs;
                sincosf(pos * a.freq[k], &sn, &cs);
                sn *= a.gain;
                cs *= a.gain;
                const float x = rows_at(a.in, t, ib + k), y = rows_at(a.in, t, ib + k + half);
                store_from_f32(a.out, a.out_dtype, ob + k, x * cs - y * sn);
                store_from_f32(a.out, a.out_dtype, ob + k + half, y * cs + x * sn);
            } else {
                const int c = 2 * half + (k - half);
                store_from_f32(a.out, a.out_dtype, ob + c, rows_at(a.in, t, ib + c));
            }
        }
    }
}

}  // namespace

// u [S][T][ld]: q_rank + kv_rank + rot columns.  cq_out [T][q_rank] and the pages in `dtype`.  A page is one flat row:
// [page_size][kv_rank + rot] key rows, then [page_size][v_width] value rows (v_width >= kv_rank; the latent, then zeros:
// value rows as wide as key rows are what the tensor-core attention kernels read).
VCB_API int vcb_latent_norm_rope_store(const float* u, int S, long long s_stride, long long ld, const float* gq, const float* gkv,
                                       float eps, const int* positions, const float* freq, float gain, const int* slot_map,
                                       void* cq_out, void* pages, long long page_stride, int page_size, int num_pages, int q_rank,
                                       int kv_rank, int rot, int v_width, int T, int dtype, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(q_rank > 0 && kv_rank > 0 && rot >= 0, "latent_norm_rope_store: bad sizes %d %d %d", q_rank, kv_rank, rot);
    VCB_CHECK_ARG(v_width >= kv_rank && v_width <= kv_rank + rot, "latent_norm_rope_store: value rows of %d lanes", v_width);
    LatentArgs a{Rows{u, S < 1 ? 1 : S, s_stride, ld}, gq, gkv, eps, positions, freq, gain, slot_map, cq_out, pages, page_stride,
                 page_size, num_pages, q_rank, kv_rank, rot, T, v_width, status};
    const size_t smem = (size_t)(q_rank + kv_rank + rot) * sizeof(float);
    VCB_CHECK_ARG(smem <= 48 * 1024, "latent_norm_rope_store: %d lanes are more than the kernel's shared memory holds", q_rank + kv_rank + rot);
    if (dtype == VCB_F32) launch_pdl(latent_norm_rope_store_kernel<float>, dim3(T), dim3(256), smem, stream, a);
    else launch_pdl(latent_norm_rope_store_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, a);
    VCB_CHECK_LAUNCH("latent_norm_rope_store");
    return 0;
}

// The same for a long step: one block is head h and HT_TOKENS tokens, a thread an output lane.  The thread walks its row of
// the matrix once (16 or 8 bytes at a time) and every token of the tile takes its sum from that pass, reading the token's
// inputs as 16-byte words that all threads share.  n_in is a multiple of four.
constexpr int HT_TOKENS = 32;

__global__ __launch_bounds__(128) void head_linear_tile_kernel(HeadLinearArgs a) {
    extern __shared__ __align__(16) float xt_s[];       // [HT_TOKENS][n_in]
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.y, t0 = blockIdx.x * HT_TOKENS;
    const int nt = min(HT_TOKENS, a.T - t0);
    for (int i = threadIdx.x; i < HT_TOKENS * a.n_in; i += blockDim.x) {
        const int tt = i / a.n_in, c = i % a.n_in;
        float v = 0.f;
        if (tt < nt) {
            const size_t at = (size_t)(t0 + tt) * a.ld_in + (size_t)h * a.in_head_stride + a.in_off + c;
            if (a.in_dtype == VCB_F32) {
                for (int s = 0; s < a.S; ++s) v += ((const float*)a.in)[at + (size_t)s * a.s_stride];
            } else {
                v = __bfloat162float(((const __nv_bfloat16*)a.in)[at]);
            }
        }
        xt_s[i] = v;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < a.n_out; j += blockDim.x) {
        float acc[HT_TOKENS];
#pragma unroll
        for (int tt = 0; tt < HT_TOKENS; ++tt) acc[tt] = 0.f;
        const size_t mrow = ((size_t)h * a.n_out + j) * a.n_in;
        for (int c = 0; c < a.n_in; c += 4) {
            float4 w;
            if (a.m_dtype == VCB_F32) {
                w = *reinterpret_cast<const float4*>((const float*)a.m + mrow + c);
            } else {
                const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)a.m + mrow + c);
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                w = make_float4(lo.x, lo.y, hi.x, hi.y);
            }
#pragma unroll
            for (int tt = 0; tt < HT_TOKENS; ++tt) {
                const float4 x = *reinterpret_cast<const float4*>(xt_s + tt * a.n_in + c);
                acc[tt] = fmaf(w.w, x.w, fmaf(w.z, x.z, fmaf(w.y, x.y, fmaf(w.x, x.x, acc[tt]))));
            }
        }
#pragma unroll
        for (int tt = 0; tt < HT_TOKENS; ++tt)
            if (tt < nt)
                store_from_f32(a.out, a.out_dtype, (size_t)(t0 + tt) * a.ld_out + (size_t)h * a.out_head_stride + a.out_off + j, acc[tt]);
    }
}

VCB_API int vcb_head_linear(const void* in, int in_dtype, int S, long long s_stride, long long ld_in, int in_head_stride, int in_off,
                            const void* m, int m_dtype, void* out, int out_dtype, long long ld_out, int out_head_stride,
                            int out_off, int T, int H, int n_in, int n_out, cudaStream_t stream) {
    if (T == 0 || H == 0 || n_out == 0) return 0;
    VCB_CHECK_ARG(in_dtype == VCB_F32 || S <= 1, "head_linear: partial sums are 32-bit");
    const size_t smem = (size_t)HL_TOKENS * n_in * sizeof(float);
    VCB_CHECK_ARG(smem <= 48 * 1024, "head_linear: %d input lanes are more than the kernel's shared memory holds", n_in);
    VCB_CHECK_ARG(H <= 65535, "head_linear: %d heads", H);
    HeadLinearArgs a{in, in_dtype, S < 1 ? 1 : S, s_stride, ld_in, in_head_stride, in_off, m, m_dtype, out, out_dtype, ld_out,
                     out_head_stride, out_off, T, H, n_in, n_out};
    const size_t tile_smem = (size_t)HT_TOKENS * n_in * sizeof(float);
    if (T >= 2 * HT_TOKENS && (n_in & 3) == 0 && tile_smem <= 48 * 1024 && (reinterpret_cast<uintptr_t>(m) & 15) == 0) {
        launch_pdl(head_linear_tile_kernel, dim3((T + HT_TOKENS - 1) / HT_TOKENS, H), dim3(128), tile_smem, stream, a);
        VCB_CHECK_LAUNCH("head_linear");
        return 0;
    }
    launch_pdl(head_linear_kernel, dim3((T + HL_TOKENS - 1) / HL_TOKENS, H), dim3(256), smem, stream, a);
    VCB_CHECK_LAUNCH("head_linear");
    return 0;
}

VCB_API int vcb_rope_rows(const float* in, int S, long long s_stride, long long ld, int in_head_stride, int in_off,
                          const int* positions, const float* freq, float gain, void* out, int out_dtype, long long ld_out,
                          int out_head_stride, int out_off, int T, int H, int dims, int width, cudaStream_t stream) {
    if (T == 0 || H == 0 || width == 0) return 0;
    VCB_CHECK_ARG(dims >= 0 && dims <= width, "rope_rows: %d rotated lanes of %d", dims, width);
    RopeArgs a{Rows{in, S < 1 ? 1 : S, s_stride, ld}, in_head_stride, in_off, positions, freq, gain, out, out_dtype, ld_out,
               out_head_stride, out_off, T, H, dims, width};
    const int per_head = dims / 2 + (width - 2 * (dims / 2));
    const dim3 grid((H * per_head + 127) / 128, T < 65535 ? T : 65535);
    launch_pdl(rope_rows_kernel, grid, dim3(128), 0, stream, a);
    VCB_CHECK_LAUNCH("rope_rows");
    return 0;
}
