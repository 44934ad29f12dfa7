// Row kernels of layers whose sublayers run side by side on one normed input, all 32-bit arithmetic on 32-bit sums or
// k-slice partial sums:
//
//  * sum_add_rmsnorm    x[t] += sum over up to four results (each maybe in k-slices) + a row of a second stream (the
//                       embedding's, where a repeated stretch of layers starts over) + a vector; out[t] = gain * x[t] /
//                       sqrt(mean(x[t]^2) + eps).  One pass over the row: the additions of everything a layer left
//                       pending and the next norm.  On a list of rows the stream itself is left alone.
//  * branch_norm_mean   out[t] = 1/N sum_b gain_b * y_b[t] / sqrt(mean(y_b[t]^2) + eps): the results of N mixers that
//                       read the same input, each normed over the model width with its own gain, averaged.
//  * polynorm           out[t] = a n(z) + b n(z^2) + c n(z^3) + e with n(v) = v / sqrt(mean(v^2) + eps) over a token's
//                       hidden lanes and powers taken lane by lane; a, b, c, e read from the device.
//
// A block a row, the row kept in shared memory between the pass that sums and the pass that writes.  Rows whose width
// and strides allow it move as 16-byte words.  The order of every sum is fixed by the width and the block size.
#include "common.cuh"

namespace {

constexpr int MAX_TERMS = 4;

struct Rows {
    const float* p;
    int S;
    long long s_stride;
    long long ld;
};

struct SumArgs {
    float* resid;               // [T][H]
    Rows term[MAX_TERMS];
    int n_terms;
    const float* row_extra;     // [T][H] or null
    const float* vec_extra;     // [H] or null
    const float* gain;          // [H] 32-bit, or null with out null
    float eps;
    void* out;                  // [n][H] or null: the additions alone
    int out_dtype;
    const int* rows;            // null: every row, and the stream is written back
    int H;
};

template <int V> struct Pack;
template <> struct Pack<1> {
    float v[1];
    __device__ __forceinline__ void load(const float* p) { v[0] = *p; }
    __device__ __forceinline__ void store(float* p) const { *p = v[0]; }
};
template <> struct Pack<4> {
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};

template <int V>
__device__ __forceinline__ void add_rows(Pack<V>& x, const Rows& in, size_t r, int c) {
    const float* p = in.p + r * in.ld + c;
    for (int s = 0; s < in.S; ++s) {
        Pack<V> t;
        t.load(p + (size_t)s * in.s_stride);
#pragma unroll
        for (int i = 0; i < V; ++i) x.v[i] += t.v[i];
    }
}

template <int V>
__device__ __forceinline__ void store_out(void* out, int dtype, size_t at, const Pack<V>& y) {
    if (dtype == VCB_F32) y.store((float*)out + at);
    else if (V == 4) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(y.v[0], y.v[V > 1 ? 1 : 0]), hi = __floats2bfloat162_rn(y.v[V > 2 ? 2 : 0], y.v[V > 3 ? 3 : 0]);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>((__nv_bfloat16*)out + at) = pk;
    } else ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(y.v[0]);
}

// N sums over the block in one round of barriers; every thread gets them all.  The order of the additions depends only
// on the block size.
template <int N>
__device__ __forceinline__ void block_sums(float (&v)[N], float* scratch /* >= N * 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = warp_sum(v[k]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < N; ++k) scratch[k * 33 + warp] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < N; ++k) {
            float t = lane < nwarps ? scratch[k * 33 + lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) scratch[k * 33 + 32] = t;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = scratch[k * 33 + 32];
}

template <int V>
__global__ __launch_bounds__(512, 3) void sum_add_rmsnorm_kernel(SumArgs a) {
    extern __shared__ __align__(16) float row_s[];      // [H]
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x, H = a.H;
    const size_t r = a.rows ? (size_t)a.rows[i] : (size_t)i;
    const bool write_back = a.rows == nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
        Pack<V> x;
        x.load(a.resid + r * H + c);
        for (int k = 0; k < a.n_terms; ++k) add_rows<V>(x, a.term[k], r, c);
        if (a.row_extra != nullptr) {
            Pack<V> t;
            t.load(a.row_extra + r * H + c);
#pragma unroll
            for (int j = 0; j < V; ++j) x.v[j] += t.v[j];
        }
        if (a.vec_extra != nullptr) {
            Pack<V> t;
            t.load(a.vec_extra + c);
#pragma unroll
            for (int j = 0; j < V; ++j) x.v[j] += t.v[j];
        }
#pragma unroll
        for (int j = 0; j < V; ++j) ss = fmaf(x.v[j], x.v[j], ss);
        if (write_back) x.store(a.resid + r * H + c);
        x.store(row_s + c);
    }
    if (a.out == nullptr) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + a.eps);
    for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
        Pack<V> x, g;
        x.load(row_s + c);
        g.load(a.gain + c);
#pragma unroll
        for (int j = 0; j < V; ++j) x.v[j] = g.v[j] * x.v[j] * inv;
        store_out<V>(a.out, a.out_dtype, (size_t)i * H + c, x);
    }
}

struct BranchArgs {
    Rows y[MAX_TERMS];
    const float* gain[MAX_TERMS];   // [H] each
    int n;
    float eps;
    float* out;                     // [T][H]
    int H;
};

template <int V>
__global__ __launch_bounds__(512, 3) void branch_norm_mean_kernel(BranchArgs a) {
    extern __shared__ __align__(16) float row_s[];      // [n][H]
    __shared__ float red[MAX_TERMS * 33];
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int H = a.H;
    float inv[MAX_TERMS];
#pragma unroll
    for (int b = 0; b < MAX_TERMS; ++b) inv[b] = 0.f;
    for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
#pragma unroll
        for (int b = 0; b < MAX_TERMS; ++b) {
            if (b < a.n) {
                Pack<V> x;
#pragma unroll
                for (int j = 0; j < V; ++j) x.v[j] = 0.f;
                add_rows<V>(x, a.y[b], t, c);
#pragma unroll
                for (int j = 0; j < V; ++j) inv[b] = fmaf(x.v[j], x.v[j], inv[b]);
                x.store(row_s + (size_t)b * H + c);
            }
        }
    }
    block_sums<MAX_TERMS>(inv, red);
#pragma unroll
    for (int b = 0; b < MAX_TERMS; ++b) inv[b] = 1.0f / sqrtf(inv[b] / (float)H + a.eps);
    const float share = 1.0f / (float)a.n;
    for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
        Pack<V> acc;
#pragma unroll
        for (int j = 0; j < V; ++j) acc.v[j] = 0.f;
        for (int b = 0; b < a.n; ++b) {
            Pack<V> x, g;
            x.load(row_s + (size_t)b * H + c);
            g.load(a.gain[b] + c);
#pragma unroll
            for (int j = 0; j < V; ++j) acc.v[j] += x.v[j] * (b == 0 ? inv[0] : b == 1 ? inv[1] : b == 2 ? inv[2] : inv[3]) * g.v[j];
        }
#pragma unroll
        for (int j = 0; j < V; ++j) acc.v[j] *= share;
        acc.store(a.out + t * H + c);
    }
}

template <int V>
__global__ __launch_bounds__(512, 3) void polynorm_kernel(Rows u, const float* __restrict__ coef, float eps, void* out, int out_dtype, int F) {
    extern __shared__ __align__(16) float row_s[];      // [F]
    __shared__ float red[3 * 33];
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int c = threadIdx.x * V; c < F; c += blockDim.x * V) {
        Pack<V> z;
#pragma unroll
        for (int j = 0; j < V; ++j) z.v[j] = 0.f;
        add_rows<V>(z, u, t, c);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float z2 = z.v[j] * z.v[j], z3 = z2 * z.v[j];
            s2 += z2;
            s4 = fmaf(z2, z2, s4);
            s6 = fmaf(z3, z3, s6);
        }
        z.store(row_s + c);
    }
    float sums[3] = {s2, s4, s6};
    block_sums<3>(sums, red);
    s2 = sums[0];
    s4 = sums[1];
    s6 = sums[2];
    const float a = coef[0], b = coef[1], cc = coef[2], e = coef[3];
    const float r1 = a / sqrtf(s2 / (float)F + eps), r2 = b / sqrtf(s4 / (float)F + eps), r3 = cc / sqrtf(s6 / (float)F + eps);
    for (int c = threadIdx.x * V; c < F; c += blockDim.x * V) {
        Pack<V> z;
        z.load(row_s + c);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float v = z.v[j], v2 = v * v;
            z.v[j] = fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e)));
        }
        store_out<V>(out, out_dtype, t * F + c, z);
    }
}

bool rows_vec_ok(const Rows& r) { return ((uintptr_t)r.p % 16 == 0) && r.ld % 4 == 0 && (r.S <= 1 || r.s_stride % 4 == 0); }

int block_for(int width, int v) {
    const int lanes = (width + v - 1) / v;
    int t = 128;
    while (t < lanes && t < 512) t <<= 1;      // (two or more blocks an SM: they hide one another's round trips)
    return t;
}

template <typename K>
int want_smem(K kern, size_t smem, const char* name) {
    if (smem > 200 * 1024) {
        vcb_set_error("%s: a row of %zu bytes is more than the kernel's shared memory holds", name, smem);
        return -1;
    }
    // (the kernels hold a few static words beside the row)
    if (smem + 1024 > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        vcb_set_error("%s: %zu bytes of shared memory refused", name, smem);
        return -2;
    }
    return 0;
}

}  // namespace

// resid [T][H]; terms: n_terms results, term k [S_k][T][ld_k] 32-bit (pointers, slice counts, slice strides, row strides in
// four arrays); row_extra [T][H] or null; vec_extra [H] or null; gain [H] 32-bit; out [n][H] of out_dtype or null (then
// only the additions are done); rows: null (every row i < n, the stream written back) or n row indices (stream untouched).
VCB_API int vcb_sum_add_rmsnorm(float* resid, int n_terms, const float* const* term_p, const int* term_S, const long long* term_ss,
                                const long long* term_ld, const float* row_extra, const float* vec_extra, const float* gain, float eps,
                                void* out, int out_dtype, const int* rows, int n, int H, cudaStream_t stream) {
    if (n == 0) return 0;
    VCB_CHECK_ARG(n_terms >= 0 && n_terms <= MAX_TERMS, "sum_add_rmsnorm: %d results at once (up to %d)", n_terms, MAX_TERMS);
    VCB_CHECK_ARG(H > 0 && (out == nullptr || gain != nullptr), "sum_add_rmsnorm: bad arguments (H=%d)", H);
    SumArgs a{};
    a.resid = resid;
    bool vec = H % 4 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)row_extra % 16 == 0 && (uintptr_t)vec_extra % 16 == 0 &&
               (uintptr_t)gain % 16 == 0 && (uintptr_t)out % 16 == 0;
    for (int k = 0; k < n_terms; ++k) {
        a.term[k] = Rows{term_p[k], term_S[k] < 1 ? 1 : term_S[k], term_ss[k], term_ld[k]};
        vec = vec && rows_vec_ok(a.term[k]);
    }
    a.n_terms = n_terms;
    a.row_extra = row_extra;
    a.vec_extra = vec_extra;
    a.gain = gain;
    a.eps = eps;
    a.out = out;
    a.out_dtype = out_dtype;
    a.rows = rows;
    a.H = H;
    const size_t smem = (size_t)H * sizeof(float);
    if (vec) {
        if (int rc = want_smem(sum_add_rmsnorm_kernel<4>, smem, "sum_add_rmsnorm")) return rc;
        launch_pdl(sum_add_rmsnorm_kernel<4>, dim3(n), dim3(block_for(H, 4)), smem, stream, a);
    } else {
        if (int rc = want_smem(sum_add_rmsnorm_kernel<1>, smem, "sum_add_rmsnorm")) return rc;
        launch_pdl(sum_add_rmsnorm_kernel<1>, dim3(n), dim3(block_for(H, 1)), smem, stream, a);
    }
    VCB_CHECK_LAUNCH("sum_add_rmsnorm");
    return 0;
}

// y_b [S_b][T][ld_b] 32-bit results of n mixers, gain_b [H]; out [T][H] 32-bit.
VCB_API int vcb_branch_norm_mean(int n, const float* const* y_p, const int* y_S, const long long* y_ss, const long long* y_ld,
                                 const float* const* gain, float eps, float* out, int T, int H, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(n >= 1 && n <= MAX_TERMS && H > 0, "branch_norm_mean: %d branches of width %d (1 to %d branches)", n, H, MAX_TERMS);
    BranchArgs a{};
    bool vec = H % 4 == 0 && (uintptr_t)out % 16 == 0;
    for (int b = 0; b < n; ++b) {
        a.y[b] = Rows{y_p[b], y_S[b] < 1 ? 1 : y_S[b], y_ss[b], y_ld[b]};
        a.gain[b] = gain[b];
        vec = vec && rows_vec_ok(a.y[b]) && (uintptr_t)gain[b] % 16 == 0;
    }
    a.n = n;
    a.eps = eps;
    a.out = out;
    a.H = H;
    const size_t smem = (size_t)n * H * sizeof(float);
    if (vec) {
        if (int rc = want_smem(branch_norm_mean_kernel<4>, smem, "branch_norm_mean")) return rc;
        launch_pdl(branch_norm_mean_kernel<4>, dim3(T), dim3(block_for(H, 4)), smem, stream, a);
    } else {
        if (int rc = want_smem(branch_norm_mean_kernel<1>, smem, "branch_norm_mean")) return rc;
        launch_pdl(branch_norm_mean_kernel<1>, dim3(T), dim3(block_for(H, 1)), smem, stream, a);
    }
    VCB_CHECK_LAUNCH("branch_norm_mean");
    return 0;
}

// u [S][T][ld] 32-bit sums of F lanes a token; coef [4] = a, b, c, e on the device; out [T][F] of out_dtype.
VCB_API int vcb_polynorm(const float* u, int S, long long s_stride, long long ld, const float* coef, float eps, void* out,
                         int out_dtype, int T, int F, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(F > 0 && coef != nullptr, "polynorm: bad arguments (F=%d)", F);
    const Rows r{u, S < 1 ? 1 : S, s_stride, ld};
    const bool vec = F % 4 == 0 && rows_vec_ok(r) && (uintptr_t)out % 16 == 0;
    const size_t smem = (size_t)F * sizeof(float);
    if (vec) {
        if (int rc = want_smem(polynorm_kernel<4>, smem, "polynorm")) return rc;
        launch_pdl(polynorm_kernel<4>, dim3(T), dim3(block_for(F, 4)), smem, stream, r, coef, eps, out, out_dtype, F);
    } else {
        if (int rc = want_smem(polynorm_kernel<1>, smem, "polynorm")) return rc;
        launch_pdl(polynorm_kernel<1>, dim3(T), dim3(block_for(F, 1)), smem, stream, r, coef, eps, out, out_dtype, F);
    }
    VCB_CHECK_LAUNCH("polynorm");
    return 0;
}
