// Rotary attention whose options are all parameters: what lies between the stacked q, k, v projection and the attention
// kernels, and the turn back behind them.
//
//  * qkv_rope_store   from a token's 32-bit sums [q | k | v] (or [q | k], where the keys as projected double as values):
//                     optionally all query lanes divided by one root mean square and multiplied by a gain per lane, the
//                     key lanes likewise; the first `rot` lanes of every q and k head turned by position * freq[i], lanes
//                     paired in halves (i, i + rot/2) or interleaved (2i, 2i+1); optionally every value head turned the
//                     same way over `vrot` of its lanes with frequencies of its own; queries to a buffer, keys and values
//                     to the token's place in the paged cache.
//  * rotate_heads     every head of a buffer turned in place by sign * position * freq[i] (the heads' weighted sums of
//                     rotated values turned back by the query's position).
//
// Norms, angles (a 32-bit product of position and frequency; the frequencies are rounded once from 64-bit on the host),
// sines and cosines are 32-bit.  A block a token; cosines and sines are computed once a token and shared by its heads.
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

struct StoreArgs {
    Rows qkv;               // [T][nh hd + nkv hd (+ nkv vd)]
    const float* q_gain;    // [nh hd] or null: no norm over the whole projection
    const float* k_gain;    // [nkv hd]
    float eps;
    const int* positions;
    const float* freq;      // [rot / 2]
    const float* vfreq;     // [vrot / 2] or null: values are stored as they are
    const int* slot_map;    // token -> page * page_size + offset, -1: stored nowhere
    void* q_out;            // [T][nh hd]
    void* pages;            // a page: [nkv][page_size][hd] keys, then [nkv][page_size][vd] values
    long long page_stride;
    int page_size, num_pages;
    int nh, nkv, hd, vd, rot, vrot;
    int interleaved;        // pairing of the rotated lanes
    int v_from_k;           // values are the key lanes as projected (before norm and rotation); vd == hd
    int* status;
};

// lanes (a, b) of pair k of a head whose first `dims` lanes turn; b < 0: lane a passes unchanged
__device__ __forceinline__ void pair_lanes(int k, int dims, int interleaved, int& a, int& b) {
    const int half = dims >> 1;
    if (k < half) {
        a = interleaved ? 2 * k : k;
        b = interleaved ? 2 * k + 1 : k + half;
    } else {
        a = dims + (k - half);
        b = -1;
    }
}

template <typename TC>
__global__ void qkv_rope_store_kernel(StoreArgs a) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int nq = a.nh * a.hd, nk = a.nkv * a.hd, nv = a.v_from_k ? 0 : a.nkv * a.vd;
    const int n = nq + nk + nv;
    float* row = sm;                    // [n]
    float* cs = sm + n;                 // [rot]: cosines, then sines
    float* vcs = cs + a.rot;            // [vrot]
    const float pos = (float)a.positions[t];
    const int half = a.rot >> 1, vhalf = a.vrot >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * a.freq[i], &cs[half + i], &cs[i]);
    if (a.vfreq != nullptr)
        for (int i = threadIdx.x; i < vhalf; i += blockDim.x) sincosf(pos * a.vfreq[i], &vcs[vhalf + i], &vcs[i]);
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = rows_at(a.qkv, t, c);
        row[c] = v;
        if (c < nq) sq = fmaf(v, v, sq);
        else if (c < nq + nk) sk = fmaf(v, v, sk);
    }
    float rq = 1.f, rk = 1.f;
    if (a.q_gain != nullptr) {
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        rq = 1.0f / sqrtf(sq / (float)nq + a.eps);
        rk = 1.0f / sqrtf(sk / (float)nk + a.eps);
    } else __syncthreads();
    // queries
    TC* q_out = (TC*)a.q_out + (size_t)t * nq;
    const int per_q = half + (a.hd - 2 * half);
    for (int i = threadIdx.x; i < a.nh * per_q; i += blockDim.x) {
        const int h = i / per_q, base = h * a.hd;
        int la, lb;
        pair_lanes(i % per_q, a.rot, a.interleaved, la, lb);
        const float x = row[base + la] * (a.q_gain ? rq * a.q_gain[base + la] : 1.f);
        if (lb < 0) q_out[base + la] = from_f32<TC>(x);
        else {
            const float y = row[base + lb] * (a.q_gain ? rq * a.q_gain[base + lb] : 1.f);
            const float c = cs[i % per_q], s = cs[half + i % per_q];
            q_out[base + la] = from_f32<TC>(x * c - y * s);
            q_out[base + lb] = from_f32<TC>(y * c + x * s);
        }
    }
    const int slot = a.slot_map[t];
    if (slot < 0) return;
    const int page = slot / a.page_size, off = slot % a.page_size;
    if (page >= a.num_pages) {
        if (threadIdx.x == 0) atomicOr(a.status, VCB_STATUS_BAD_PAGE);
        return;
    }
    TC* kp = (TC*)a.pages + (size_t)page * a.page_stride;
    TC* vp = kp + (size_t)a.nkv * a.page_size * a.hd;
    // keys
    for (int i = threadIdx.x; i < a.nkv * per_q; i += blockDim.x) {
        const int g = i / per_q, base = nq + g * a.hd;
        TC* dst = kp + ((size_t)g * a.page_size + off) * a.hd;
        int la, lb;
        pair_lanes(i % per_q, a.rot, a.interleaved, la, lb);
        const float x = row[base + la] * (a.k_gain ? rk * a.k_gain[g * a.hd + la] : 1.f);
        if (lb < 0) dst[la] = from_f32<TC>(x);
        else {
            const float y = row[base + lb] * (a.k_gain ? rk * a.k_gain[g * a.hd + lb] : 1.f);
            const float c = cs[i % per_q], s = cs[half + i % per_q];
            dst[la] = from_f32<TC>(x * c - y * s);
            dst[lb] = from_f32<TC>(y * c + x * s);
        }
    }
    // values
    const int vr = a.vfreq != nullptr ? a.vrot : 0;
    const int per_v = (vr >> 1) + (a.vd - 2 * (vr >> 1));
    for (int i = threadIdx.x; i < a.nkv * per_v; i += blockDim.x) {
        const int g = i / per_v, base = a.v_from_k ? nq + g * a.hd : nq + nk + g * a.vd;
        TC* dst = vp + ((size_t)g * a.page_size + off) * a.vd;
        int la, lb;
        pair_lanes(i % per_v, vr, a.interleaved, la, lb);
        const float x = row[base + la];
        if (lb < 0) dst[la] = from_f32<TC>(x);
        else {
            const float y = row[base + lb];
            const float c = vcs[i % per_v], s = vcs[vhalf + i % per_v];
            dst[la] = from_f32<TC>(x * c - y * s);
            dst[lb] = from_f32<TC>(y * c + x * s);
        }
    }
}

template <typename TC>
__global__ void rotate_heads_kernel(TC* x, const int* __restrict__ positions, const float* __restrict__ freq, float sign, int H,
                                    int width, int dims, int interleaved) {
    extern __shared__ float cs[];       // [dims]
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, half = dims >> 1;
    const float pos = sign * (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * freq[i], &cs[half + i], &cs[i]);
    __syncthreads();
    TC* row = x + (size_t)t * H * width;
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, k = i % half;
        int la, lb;
        pair_lanes(k, dims, interleaved, la, lb);
        TC* p = row + (size_t)h * width;
        const float u = to_f32(p[la]), v = to_f32(p[lb]);
        p[la] = from_f32<TC>(u * cs[k] - v * cs[half + k]);
        p[lb] = from_f32<TC>(v * cs[k] + u * cs[half + k]);
    }
}

}  // namespace

// qkv [S][T][ld] 32-bit sums; q_out [T][nh hd] and the pages of `dtype`; vfreq null: values stored unturned.
VCB_API int vcb_qkv_rope_store(const float* qkv, int S, long long s_stride, long long ld, const float* q_gain, const float* k_gain,
                               float eps, const int* positions, const float* freq, const float* vfreq, const int* slot_map,
                               void* q_out, void* pages, long long page_stride, int page_size, int num_pages, int nh, int nkv,
                               int hd, int vd, int rot, int vrot, int interleaved, int v_from_k, int T, int dtype, int* status,
                               cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && hd > 0 && vd > 0, "qkv_rope_store: bad sizes %d %d %d %d", nh, nkv, hd, vd);
    VCB_CHECK_ARG(rot >= 0 && rot <= hd && rot % 2 == 0, "qkv_rope_store: %d turning lanes of %d", rot, hd);
    VCB_CHECK_ARG(vfreq == nullptr || (vrot >= 0 && vrot <= vd && vrot % 2 == 0), "qkv_rope_store: %d turning value lanes of %d", vrot, vd);
    VCB_CHECK_ARG(!v_from_k || vd == hd, "qkv_rope_store: keys that double as values have their size (%d, not %d)", hd, vd);
    VCB_CHECK_ARG((q_gain == nullptr) == (k_gain == nullptr), "qkv_rope_store: one gain without the other");
    VCB_CHECK_ARG(rot == 0 || freq != nullptr, "qkv_rope_store: no frequencies");
    StoreArgs a{Rows{qkv, S < 1 ? 1 : S, s_stride, ld}, q_gain, k_gain, eps, positions, freq, vfreq, slot_map, q_out, pages, page_stride,
                page_size, num_pages, nh, nkv, hd, vd, rot, vfreq ? vrot : 0, interleaved, v_from_k, status};
    const size_t smem = (size_t)(nh * hd + nkv * hd + (v_from_k ? 0 : nkv * vd) + rot + (vfreq ? vrot : 0)) * sizeof(float);
    VCB_CHECK_ARG(smem <= 200 * 1024, "qkv_rope_store: a token's %zu bytes are more than the kernel's shared memory holds", smem);
    auto kern = dtype == VCB_F32 ? qkv_rope_store_kernel<float> : qkv_rope_store_kernel<__nv_bfloat16>;
    if (smem + 1024 > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        vcb_set_error("qkv_rope_store: %zu bytes of shared memory refused", smem);
        return -2;
    }
    launch_pdl(kern, dim3(T), dim3(256), smem, stream, a);
    VCB_CHECK_LAUNCH("qkv_rope_store");
    return 0;
}

// x [T][H][width] of `dtype`, in place: the first `dims` lanes of every head turn by sign * position * freq[i].
VCB_API int vcb_rotate_heads(void* x, int dtype, const int* positions, const float* freq, float sign, int T, int H, int width,
                             int dims, int interleaved, cudaStream_t stream) {
    if (T == 0 || H == 0 || dims == 0) return 0;
    VCB_CHECK_ARG(dims > 0 && dims <= width && dims % 2 == 0, "rotate_heads: %d turning lanes of %d", dims, width);
    const size_t smem = (size_t)dims * sizeof(float);
    const int threads = H * dims / 2 >= 256 ? 256 : 128;
    if (dtype == VCB_F32)
        launch_pdl(rotate_heads_kernel<float>, dim3(T), dim3(threads), smem, stream, (float*)x, positions, freq, sign, H, width, dims, interleaved);
    else
        launch_pdl(rotate_heads_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, (__nv_bfloat16*)x, positions, freq, sign, H, width,
                   dims, interleaved);
    VCB_CHECK_LAUNCH("rotate_heads");
    return 0;
}
