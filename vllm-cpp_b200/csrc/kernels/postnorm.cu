// Kernels of layers that norm a sublayer's result before it is added, and the small steps around them:
//
//  * embed_scaled_pos     x[t] = s * E[id_t] + P[p_t]          (a learned vector per position, not scaled)
//  * postnorm_add_norm    x_t += l * (w_b * n(y_t + b));  out_t = w_n * n'(x_t)
//                         n(v) = v / sqrt(mean(v^2) + eps): the norm on what a sublayer returned, an optional
//                         per-channel layer scale l, the addition into the 32-bit stream, and the norm in front of
//                         the next sublayer -- one kernel, one pass over the row
//  * qkv_wholenorm_store  the stacked q, k, v projection; all of a token's query lanes divided by their common
//                         root mean square and multiplied by a gain per lane (no split into heads first), the
//                         same for its key lanes; queries to a buffer, keys and values to the tokens' cache slots
//  * gated_act            act(g + b_g) * (u + b_u) for a feed-forward with a gate beside its up projection
//  * softcap              z <- c * tanh(z / c) in place (capped logits)
//
// All arithmetic is 32-bit; inputs that are matrix products arrive as 32-bit sums, possibly as k-slice partial sums
// [S, T, C] that are added here in slice order.  Rows beyond every entry (padding of a captured step) are left alone.
#include "common.cuh"

namespace {

__device__ __forceinline__ int entry_of_row(const int* __restrict__ q_start, const int* __restrict__ q_len, int E, int t) {
    int lo = 0, hi = E;   // first index with q_start > t
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (q_start[mid] <= t) lo = mid + 1;
        else hi = mid;
    }
    const int e = lo - 1;
    if (e < 0) return -1;
    return t - q_start[e] < q_len[e] ? e : -1;
}

struct Rows {
    const float* p;       // [S][T][ld] 32-bit sums
    int S;
    long long s_stride;   // elements between partial sums
    long long ld;         // elements between rows
    const float* bias;    // [C] or null
};

__device__ __forceinline__ float rows_at(const Rows& in, long long t, int c) {
    float v = 0.f;
    const float* p = in.p + t * in.ld + c;
    for (int s = 0; s < in.S; ++s) v += p[(long long)s * in.s_stride];
    if (in.bias != nullptr) v += in.bias[c];
    return v;
}

// four neighbouring channels at once (c a multiple of 4, every stride and base a multiple of 4 elements)
__device__ __forceinline__ float4 rows_at4(const Rows& in, long long t, int c) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* p = in.p + t * in.ld + c;
    for (int s = 0; s < in.S; ++s) {
        const float4 a = *reinterpret_cast<const float4*>(p + (long long)s * in.s_stride);
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
    }
    if (in.bias != nullptr) {
        const float4 b = *reinterpret_cast<const float4*>(in.bias + c);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    }
    return v;
}
inline bool rows_vec_ok(const Rows& r) {
    return r.p == nullptr || (((uintptr_t)r.p % 16 == 0) && r.ld % 4 == 0 && (r.S <= 1 || r.s_stride % 4 == 0) &&
                              (r.bias == nullptr || (uintptr_t)r.bias % 16 == 0));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ float act_of(float x, int kind) {
    switch (kind) {
        case 0: return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
        case 1: return 0.5f * x * (1.f + tanhf(0.79788456080286535588f * (x + 0.044715f * x * x * x)));
        case 2: return x / (1.f + expf(-x));
        case 3: { const float r = fmaxf(x, 0.f); return r * r; }
        default: return x;
    }
}

__global__ void embed_scaled_pos_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ ids,
                                        const int* __restrict__ positions, const void* __restrict__ pos_table, int pos_dtype,
                                        float scale, float* __restrict__ out, int H, int V, int P, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t], p = pos_table != nullptr ? positions[t] : 0;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && status != nullptr) atomicOr(status, VCB_STATUS_BAD_TOKEN);
        id = 0;
    }
    if (pos_table == nullptr) {
        // no position vectors: the scaled row alone
        for (int c = threadIdx.x; c < H; c += blockDim.x)
            out[(size_t)t * H + c] = load_as_f32(table, table_dtype, (size_t)id * H + c) * scale;
        return;
    }
    if (p < 0 || p >= P) {
        if (threadIdx.x == 0 && status != nullptr) atomicOr(status, VCB_STATUS_BAD_POSITION);
        p = 0;
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[(size_t)t * H + c] = fmaf(load_as_f32(table, table_dtype, (size_t)id * H + c), scale,
                                      load_as_f32(pos_table, pos_dtype, (size_t)p * H + c));
}

// A block a row.  The row's values stay in shared memory between the passes.  With `rows` the kernel takes the
// listed rows only, leaves the stream alone and writes its output compactly (the rows whose logits are wanted).
template <typename TOUT>
__global__ void postnorm_add_norm_kernel(float* __restrict__ resid, Rows y, const float* __restrict__ wb,
                                         const float* __restrict__ ls, float eps_b, const int* __restrict__ q_start,
                                         const int* __restrict__ q_len, int E, int H, const float* __restrict__ wn,
                                         float eps_n, TOUT* __restrict__ out, const int* __restrict__ rows) {
    extern __shared__ float vals[];   // [H] then 33 floats for the block sum
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x;
    const long long t = rows != nullptr ? rows[i] : i;
    if (rows == nullptr && entry_of_row(q_start, q_len, E, (int)t) < 0) return;
    float ss = 0.f;
    if (y.p != nullptr) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = rows_at(y, t, c);
            vals[c] = v;
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, vals + H);
    }
    const float mul = 1.f / sqrtf(ss / (float)H + eps_b);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x = resid[(size_t)t * H + c];
        if (y.p != nullptr) {
            float d = vals[c] * mul * wb[c];
            if (ls != nullptr) d *= ls[c];
            x += d;
            if (rows == nullptr) resid[(size_t)t * H + c] = x;
        }
        vals[c] = x;
        s2 = fmaf(x, x, s2);
    }
    if (out == nullptr) return;
    s2 = block_sum(s2, vals + H);
    const float mul2 = 1.f / sqrtf(s2 / (float)H + eps_n);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[(size_t)i * H + c] = from_f32<TOUT>(vals[c] * mul2 * wn[c]);
}

// the same with four channels a thread and the row held in registers: every load of the row is asked for before the
// first result is needed
template <typename TOUT, int VPT>
__global__ __launch_bounds__(1024) void postnorm_add_norm_vec_kernel(float* __restrict__ resid, Rows y, const float* __restrict__ wb,
                                                                     const float* __restrict__ ls, float eps_b,
                                                                     const int* __restrict__ q_start, const int* __restrict__ q_len,
                                                                     int E, int H, const float* __restrict__ wn, float eps_n,
                                                                     TOUT* __restrict__ out, const int* __restrict__ rows) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x;
    const long long t = rows != nullptr ? rows[i] : i;
    if (rows == nullptr && entry_of_row(q_start, q_len, E, (int)t) < 0) return;
    const int nv = H >> 2;
    float4 v[VPT], r[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int idx = threadIdx.x + k * blockDim.x;
        if (idx < nv) {
            r[k] = *reinterpret_cast<const float4*>(resid + (size_t)t * H + 4 * idx);
            if (y.p != nullptr) v[k] = rows_at4(y, t, 4 * idx);
        }
    }
    float mul = 0.f;
    if (y.p != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k)
            if (threadIdx.x + k * blockDim.x < nv) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        ss = block_sum(ss, scratch);
        mul = 1.f / sqrtf(ss / (float)H + eps_b);
    }
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int idx = threadIdx.x + k * blockDim.x;
        if (idx < nv) {
            if (y.p != nullptr) {
                float4 d = *reinterpret_cast<const float4*>(wb + 4 * idx);
                d.x *= v[k].x * mul; d.y *= v[k].y * mul; d.z *= v[k].z * mul; d.w *= v[k].w * mul;
                if (ls != nullptr) {
                    const float4 l = *reinterpret_cast<const float4*>(ls + 4 * idx);
                    d.x *= l.x; d.y *= l.y; d.z *= l.z; d.w *= l.w;
                }
                r[k].x += d.x; r[k].y += d.y; r[k].z += d.z; r[k].w += d.w;
                if (rows == nullptr) *reinterpret_cast<float4*>(resid + (size_t)t * H + 4 * idx) = r[k];
            }
            s2 += r[k].x * r[k].x + r[k].y * r[k].y + r[k].z * r[k].z + r[k].w * r[k].w;
        }
    }
    if (out == nullptr) return;
    s2 = block_sum(s2, scratch);
    const float mul2 = 1.f / sqrtf(s2 / (float)H + eps_n);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int idx = threadIdx.x + k * blockDim.x;
        if (idx < nv) {
            const float4 g = *reinterpret_cast<const float4*>(wn + 4 * idx);
            store4<TOUT>(out + (size_t)i * H + 4 * idx, make_float4(r[k].x * mul2 * g.x, r[k].y * mul2 * g.y, r[k].z * mul2 * g.z, r[k].w * mul2 * g.w));
        }
    }
}

struct QkvWholeArgs {
    Rows in;
    const float* qw;      // [nh * hd] gain of the query lanes, or null: no norm
    const float* kw;      // [nkv * hd]
    float eps;
    const int* q_start;
    const int* q_len;
    const int* slot_map;  // [T]: page * page_size + offset of the token's cache entry, -1: none
    int E, nh, nkv, hd, hd_v;
    void* q_out;          // [T][nh * hd]
    void* pages;
    long long page_stride;
    int page_size, num_pages;
    int* status;
};

// a block a row: the row's sums in shared memory, the two sums of squares, then the stores
template <typename TOUT>
__global__ void qkv_wholenorm_store_kernel(QkvWholeArgs a) {
    extern __shared__ float vals[];   // [C] then 33 floats
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if (entry_of_row(a.q_start, a.q_len, a.E, t) < 0) return;
    const int nq = a.nh * a.hd, nk = a.nkv * a.hd, nv = a.nkv * a.hd_v;
    const int C = nq + nk + nv;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float v = rows_at(a.in, t, c);
        vals[c] = v;
        if (c < nq) sq = fmaf(v, v, sq);
        else if (c < nq + nk) sk = fmaf(v, v, sk);
    }
    float mq = 1.f, mk = 1.f;
    if (a.qw != nullptr) {
        sq = block_sum(sq, vals + C);
        sk = block_sum(sk, vals + C);
        mq = 1.f / sqrtf(sq / (float)nq + a.eps);
        mk = 1.f / sqrtf(sk / (float)nk + a.eps);
    } else {
        __syncthreads();
    }
    long long slot = a.slot_map[t];
    if (slot >= (long long)a.num_pages * a.page_size) {
        if (threadIdx.x == 0 && a.status != nullptr) atomicOr(a.status, VCB_STATUS_BAD_PAGE);
        slot = -1;
    }
    TOUT* q_out = reinterpret_cast<TOUT*>(a.q_out) + (size_t)t * nq;
    TOUT* page = slot >= 0 ? reinterpret_cast<TOUT*>(a.pages) + (slot / a.page_size) * a.page_stride : nullptr;
    const long long off = slot >= 0 ? slot % a.page_size : 0;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float v = vals[c];
        if (c < nq) {
            q_out[c] = from_f32<TOUT>(a.qw != nullptr ? v * mq * a.qw[c] : v);
        } else if (page != nullptr) {
            if (c < nq + nk) {
                const int j = c - nq, kvh = j / a.hd, d = j % a.hd;
                page[((long long)kvh * a.page_size + off) * a.hd + d] = from_f32<TOUT>(a.kw != nullptr ? v * mk * a.kw[j] : v);
            } else {
                const int j = c - nq - nk, kvh = j / a.hd_v, d = j % a.hd_v;
                page[(long long)a.nkv * a.page_size * a.hd + ((long long)kvh * a.page_size + off) * a.hd_v + d] = from_f32<TOUT>(v);
            }
        }
    }
}

// in: [S][T][2 I] sums, the gate's I columns first, then the up projection's; bias [2 I] or null
template <typename TOUT>
__global__ void gated_act_kernel(Rows in, TOUT* __restrict__ out, int T, int I, int kind) {
    pdl_trigger();
    pdl_wait();
    for (int t = blockIdx.y; t < T; t += gridDim.y)
        for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < I; c += gridDim.x * blockDim.x)
            out[(size_t)t * I + c] = from_f32<TOUT>(act_of(rows_at(in, t, c), kind) * rows_at(in, t, I + c));
}

__global__ void softcap_kernel(float* __restrict__ z, long long n, float cap) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        z[i] = cap * tanhf(z[i] / cap);
}

template <typename K>
int raise_smem(K kern, size_t smem, const char* name) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        vcb_set_error("%s: %zu bytes of shared memory refused", name, smem);
        return -2;
    }
    return 0;
}

}  // namespace

VCB_API int vcb_embed_scaled_pos(const void* table, int table_dtype, const int* ids, const int* positions,
                                 const void* pos_table, int pos_dtype, float scale, float* out, int T, int H, int V, int P,
                                 int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(H > 0 && V > 0 && (P > 0 || pos_table == nullptr), "embed_scaled_pos: bad sizes H=%d V=%d P=%d", H, V, P);
    launch_pdl(embed_scaled_pos_kernel, dim3(T), dim3(256), 0, stream, table, table_dtype, ids, positions, pos_table, pos_dtype,
               scale, out, H, V, P, status);
    VCB_CHECK_LAUNCH("embed_scaled_pos");
    return 0;
}

// y (or null: nothing is added): the sublayer's result [Sy][T][ldy] with bias yb; wb: the gain of the norm on it; ls: a
// layer scale per channel or null.  wn / out (or null): the gain of the next norm and where its rows go, in out_dtype.
// rows (or null): n_rows row indices; the stream is then left as it is and out is [n_rows][H].
VCB_API int vcb_postnorm_add_norm(float* resid, const float* y, int Sy, long long y_stride, long long ldy, const float* yb,
                                  const float* wb, const float* ls, float eps_b, const int* q_start, const int* q_len, int E,
                                  int T, int H, const float* wn, float eps_n, void* out, int out_dtype, const int* rows,
                                  int n_rows, cudaStream_t stream) {
    const int n = rows != nullptr ? n_rows : T;
    if (n == 0) return 0;
    VCB_CHECK_ARG(y == nullptr || wb != nullptr, "postnorm_add_norm: a result to add needs the gain of its norm");
    VCB_CHECK_ARG((out == nullptr) == (wn == nullptr), "postnorm_add_norm: the next norm needs both its gain and its output");
    Rows ry{y, Sy < 1 ? 1 : Sy, y_stride, ldy, yb};
    if (H % 4 == 0 && H / 4 <= 4096 && rows_vec_ok(ry) && (uintptr_t)resid % 16 == 0 && (uintptr_t)wb % 16 == 0 && (uintptr_t)ls % 16 == 0 &&
        (uintptr_t)wn % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const int nv = H / 4;
        const int vpt = nv <= 512 ? 1 : (nv <= 2048 ? 2 : 4);     // (two blocks of 512 threads fit an SM)
        const int threads4 = ((nv + vpt - 1) / vpt + 31) / 32 * 32;
#define VCB_PNA(TOUT, V) launch_pdl(postnorm_add_norm_vec_kernel<TOUT, V>, dim3(n), dim3(threads4), 0, stream, resid, ry, wb, ls, eps_b, q_start, q_len, E, H, wn, eps_n, (TOUT*)out, rows)
        if (out_dtype == VCB_F32) { if (vpt == 1) VCB_PNA(float, 1); else if (vpt == 2) VCB_PNA(float, 2); else VCB_PNA(float, 4); }
        else { if (vpt == 1) VCB_PNA(__nv_bfloat16, 1); else if (vpt == 2) VCB_PNA(__nv_bfloat16, 2); else VCB_PNA(__nv_bfloat16, 4); }
#undef VCB_PNA
        VCB_CHECK_LAUNCH("postnorm_add_norm");
        return 0;
    }
    const size_t smem = ((size_t)H + 64) * sizeof(float);
    const int threads = H >= 4096 ? 1024 : (H >= 1024 ? 512 : 256);
    if (out_dtype == VCB_F32) {
        auto kern = postnorm_add_norm_kernel<float>;
        if (int rc = raise_smem(kern, smem, "postnorm_add_norm")) return rc;
        launch_pdl(kern, dim3(n), dim3(threads), smem, stream, resid, ry, wb, ls, eps_b, q_start, q_len, E, H, wn, eps_n, (float*)out, rows);
    } else {
        auto kern = postnorm_add_norm_kernel<__nv_bfloat16>;
        if (int rc = raise_smem(kern, smem, "postnorm_add_norm")) return rc;
        launch_pdl(kern, dim3(n), dim3(threads), smem, stream, resid, ry, wb, ls, eps_b, q_start, q_len, E, H, wn, eps_n, (__nv_bfloat16*)out, rows);
    }
    VCB_CHECK_LAUNCH("postnorm_add_norm");
    return 0;
}

// in: [S][T][ld] sums of the stacked projection, C = nh hd + nkv (hd + hd_v).  qw, kw: gains over all query lanes and
// all key lanes (both or neither).  A page holds [nkv][page_size][hd] keys followed by [nkv][page_size][hd_v] values.
VCB_API int vcb_qkv_wholenorm_store(const float* in, int S, long long s_stride, long long ld, const float* qw, const float* kw,
                                    float eps, const int* q_start, const int* q_len, const int* slot_map, int E, int T, int nh,
                                    int nkv, int hd, int hd_v, void* q_out, void* pages, long long page_stride, int page_size,
                                    int num_pages, int out_dtype, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG((qw == nullptr) == (kw == nullptr), "qkv_wholenorm_store: the norm needs the gains of queries and keys");
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && hd > 0 && hd_v > 0 && page_size > 0, "qkv_wholenorm_store: bad sizes");
    QkvWholeArgs a{Rows{in, S < 1 ? 1 : S, s_stride, ld, nullptr}, qw, kw, eps, q_start, q_len, slot_map, E, nh, nkv, hd, hd_v,
                   q_out, pages, page_stride, page_size, num_pages, status};
    const int C = nh * hd + nkv * (hd + hd_v);
    const size_t smem = ((size_t)C + 64) * sizeof(float);
    const int threads = C >= 4096 ? 1024 : (C >= 1024 ? 512 : 256);
    if (out_dtype == VCB_F32) {
        auto kern = qkv_wholenorm_store_kernel<float>;
        if (int rc = raise_smem(kern, smem, "qkv_wholenorm_store")) return rc;
        launch_pdl(kern, dim3(T), dim3(threads), smem, stream, a);
    } else {
        auto kern = qkv_wholenorm_store_kernel<__nv_bfloat16>;
        if (int rc = raise_smem(kern, smem, "qkv_wholenorm_store")) return rc;
        launch_pdl(kern, dim3(T), dim3(threads), smem, stream, a);
    }
    VCB_CHECK_LAUNCH("qkv_wholenorm_store");
    return 0;
}

// kind 0: GELU with erf, 1: GELU with tanh, 2: SiLU, 3: the square of ReLU
VCB_API int vcb_gated_act(const float* in, int S, long long s_stride, long long ld, const float* bias, void* out, int out_dtype,
                          int T, int I, int kind, cudaStream_t stream) {
    if (T == 0 || I == 0) return 0;
    VCB_CHECK_ARG(kind >= 0 && kind <= 3, "gated_act: unknown activation %d", kind);
    Rows r{in, S < 1 ? 1 : S, s_stride, ld, bias};
    const dim3 grid((I + 255) / 256, T < 65535 ? T : 65535);
    if (out_dtype == VCB_F32) launch_pdl(gated_act_kernel<float>, grid, dim3(256), 0, stream, r, (float*)out, T, I, kind);
    else launch_pdl(gated_act_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, r, (__nv_bfloat16*)out, T, I, kind);
    VCB_CHECK_LAUNCH("gated_act");
    return 0;
}

VCB_API int vcb_softcap(float* z, long long n, float cap, cudaStream_t stream) {
    if (n == 0) return 0;
    VCB_CHECK_ARG(cap > 0.f, "softcap: the cap must be positive");
    const long long blocks = (n + 255) / 256;
    launch_pdl(softcap_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream, z, n, cap);
    VCB_CHECK_LAUNCH("softcap");
    return 0;
}
