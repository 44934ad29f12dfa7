// Kernels of layers that mix a few neighbouring tokens per channel and gate what a sublayer returns:
//
//  * embed_sinusoid      x[t] = E[id_t] + s(p_t),  s(p)[2i] = sin(p f_i),  s(p)[2i+1] = cos(p f_i)
//  * causal_conv         y_t = sum_j w[:, j] u_(t - taps + 1 + j)  per channel, u = 0 before a request's first token;
//                        the taps - 1 inputs before a portion come from the request's state row
//  * conv_state_update   the state row afterwards: the last taps - 1 inputs the request has seen (entries of one
//                        token are brought up to date by the convolving kernel itself: a step of single tokens
//                        launches no update)
//  * qkv_conv_norm_store the same convolution on the stacked q, k, v projection (with its bias), then every query
//                        and key head divided by its root mean square, queries to a buffer, keys and values to
//                        the tokens' cache slots
//  * gated_norm_add      x_t += w * n(y_t * sigmoid(g_t + b)),  n(v) = v / sqrt(mean(v^2) + eps)
//  * bias_act            act(u + b) for the feed-forward's hidden layer (erf or tanh GELU)
//
// All arithmetic is 32-bit; inputs that are matrix products arrive as 32-bit sums, possibly as k-slice partial sums
// [S, T, C] that are added here in slice order.  A step's rows belong to entries (q_start, q_len per entry, rows in
// entry order); rows beyond every entry (padding of a captured step) are left alone.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

// the entry a row belongs to, or -1: the last entry that starts at or before the row (entries without tokens share
// their start with the one after them, so the last of equals is the one that has the row)
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

struct RowsIn {
    const float* p;       // [S][T][ld] 32-bit sums
    int S;
    long long s_stride;   // elements between partial sums
    long long ld;         // elements between rows
    const float* bias;    // [C] or null
};

__device__ __forceinline__ float rows_at(const RowsIn& in, long long t, int c) {
    float v = 0.f;
    const float* p = in.p + t * in.ld + c;
    for (int s = 0; s < in.S; ++s) v += p[(long long)s * in.s_stride];
    if (in.bias != nullptr) v += in.bias[c];
    return v;
}

// the same for four neighbouring channels at once (c a multiple of 4, every stride and base a multiple of 4 elements)
__device__ __forceinline__ float4 rows_at4(const RowsIn& in, long long t, int c) {
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

__device__ __forceinline__ float4 conv_at4(const RowsIn& in, const float* __restrict__ w, const float* __restrict__ st, int C,
                                           int taps, long long t, int rel, int c) {
    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float4 u = rel - back >= 0 ? rows_at4(in, t - back, c) : *reinterpret_cast<const float4*>(st + (long long)(rel + j) * C + c);
        const float* wc = w + (long long)c * taps + j;
        y.x = fmaf(wc[0], u.x, y.x);
        y.y = fmaf(wc[taps], u.y, y.y);
        y.z = fmaf(wc[2 * taps], u.z, y.z);
        y.w = fmaf(wc[3 * taps], u.w, y.w);
    }
    return y;
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

// whether rows can be read four channels at a time
inline bool rows_vec_ok(const RowsIn& r) {
    return r.p == nullptr || (((uintptr_t)r.p % 16 == 0) && r.ld % 4 == 0 && (r.S <= 1 || r.s_stride % 4 == 0) &&
                              (r.bias == nullptr || (uintptr_t)r.bias % 16 == 0));
}

// sum_j w[c][j] * u(rel - taps + 1 + j) for the row at place `rel` of its entry (row index t); places before the
// entry's first row come from the state row st[k][c], k = place + taps - 1
__device__ __forceinline__ float conv_at(const RowsIn& in, const float* __restrict__ w, const float* __restrict__ st, int C,
                                         int taps, long long t, int rel, int c) {
    float y = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float u = rel - back >= 0 ? rows_at(in, t - back, c) : st[(long long)(rel + j) * C + c];
        y = fmaf(w[(long long)c * taps + j], u, y);
    }
    return y;
}

// The state row of an entry that brought one token: its rows move up by one and the token's input is the last.  Done
// by the thread that convolved the channel, after its own reads: with one token the entry has no other reader, so the
// update needs no kernel of its own (conv_state_update leaves such entries out).
__device__ __forceinline__ void state_push(float* __restrict__ st, int C, int taps, int c, float u) {
    float old[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) old[k] = k + 1 < taps - 1 ? st[(long long)(k + 1) * C + c] : 0.f;
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k)
        if (k + 1 < taps - 1) st[(long long)k * C + c] = old[k];
    st[(long long)(taps - 2) * C + c] = u;
}
__device__ __forceinline__ void state_push4(float* __restrict__ st, int C, int taps, int c, float4 u) {
    float4 old[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k)
        old[k] = k + 1 < taps - 1 ? *reinterpret_cast<const float4*>(st + (long long)(k + 1) * C + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k)
        if (k + 1 < taps - 1) *reinterpret_cast<float4*>(st + (long long)k * C + c) = old[k];
    *reinterpret_cast<float4*>(st + (long long)(taps - 2) * C + c) = u;
}

__global__ void embed_sinusoid_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ ids,
                                      const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                      float* __restrict__ out, int H, int V, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && status != nullptr) atomicOr(status, VCB_STATUS_BAD_TOKEN);
        id = 0;
    }
    const float p = (float)positions[t];
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float ang = p * inv_freq[c >> 1];
        const float s = (c & 1) ? cosf(ang) : sinf(ang);
        out[(size_t)t * H + c] = load_as_f32(table, table_dtype, (size_t)id * H + c) + s;
    }
}

template <typename TOUT>
__global__ void causal_conv_kernel(RowsIn in, const float* __restrict__ w, float* __restrict__ state,
                                   long long slot_stride, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ slots, int E, int T, int C, int taps, int add_input,
                                   TOUT* __restrict__ out_conv, TOUT* __restrict__ out_copy, const float* __restrict__ out_bias,
                                   int act) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int e = entry_of_row(q_start, q_len, E, t);
    if (e < 0) return;
    const float u = rows_at(in, t, c);
    if (out_copy != nullptr) out_copy[(size_t)t * C + c] = from_f32<TOUT>(u);
    if (out_conv != nullptr) {
        float y = taps > 0 ? conv_at(in, w, state + (long long)slots[e] * slot_stride, C, taps, t, t - q_start[e], c) : 0.f;
        if (add_input) y += u;
        if (out_bias != nullptr) y += out_bias[c];
        if (act == 1) y = y / (1.f + expf(-y));
        out_conv[(size_t)t * C + c] = from_f32<TOUT>(y);
    }
    if (taps > 1 && q_len[e] == 1) state_push(state + (long long)slots[e] * slot_stride, C, taps, c, u);
}

// four channels a thread
template <typename TOUT>
__global__ void causal_conv_vec_kernel(RowsIn in, const float* __restrict__ w, float* __restrict__ state,
                                       long long slot_stride, const int* __restrict__ q_start, const int* __restrict__ q_len,
                                       const int* __restrict__ slots, int E, int T, int C, int taps, int add_input,
                                       TOUT* __restrict__ out_conv, TOUT* __restrict__ out_copy,
                                       const float* __restrict__ out_bias, int act) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (c >= C) return;
    const int e = entry_of_row(q_start, q_len, E, t);
    if (e < 0) return;
    const float4 u = rows_at4(in, t, c);
    if (out_copy != nullptr) store4<TOUT>(out_copy + (size_t)t * C + c, u);
    if (out_conv != nullptr) {
        float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
        if (taps > 0) y = conv_at4(in, w, state + (long long)slots[e] * slot_stride, C, taps, t, t - q_start[e], c);
        if (add_input) { y.x += u.x; y.y += u.y; y.z += u.z; y.w += u.w; }
        if (out_bias != nullptr) {
            const float4 b = *reinterpret_cast<const float4*>(out_bias + c);
            y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w;
        }
        if (act == 1) {
            y.x = y.x / (1.f + expf(-y.x)); y.y = y.y / (1.f + expf(-y.y));
            y.z = y.z / (1.f + expf(-y.z)); y.w = y.w / (1.f + expf(-y.w));
        }
        store4<TOUT>(out_conv + (size_t)t * C + c, y);
    }
    if (taps > 1 && q_len[e] == 1) state_push4(state + (long long)slots[e] * slot_stride, C, taps, c, u);
}

// The same for steps of many rows: a thread walks a run of RUN rows for its four channels and keeps the window of the last
// inputs in registers, so every input row is fetched once (not once per tap) and the entry is looked up once per run (or
// where a row leaves it).  The window and the taps are held right-aligned in MAX_TAPS places, the unused older ones zero:
// the sum runs over them from the oldest to the newest, which is the order conv_at4 adds in.
template <typename TOUT, int RUN>
__global__ __launch_bounds__(128) void causal_conv_run_kernel(RowsIn in, const float* __restrict__ w, float* __restrict__ state,
                                                              long long slot_stride, const int* __restrict__ q_start,
                                                              const int* __restrict__ q_len, const int* __restrict__ slots, int E, int T,
                                                              int C, int taps, int add_input, TOUT* __restrict__ out_conv,
                                                              TOUT* __restrict__ out_copy, const float* __restrict__ out_bias, int act) {
    pdl_trigger();
    pdl_wait();
    const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (c >= C) return;
    const int t0 = blockIdx.y * RUN, t1 = min(T, t0 + RUN);
    float wr[4][MAX_TAPS];
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int b = 0; b < MAX_TAPS; ++b) wr[k][MAX_TAPS - 1 - b] = b < taps ? w[(long long)(c + k) * taps + (taps - 1 - b)] : 0.f;
    float4 ob = make_float4(0.f, 0.f, 0.f, 0.f);
    if (out_bias != nullptr) ob = *reinterpret_cast<const float4*>(out_bias + c);
    float4 win[MAX_TAPS];      // win[MAX_TAPS - 1 - b]: the input b rows back
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i) win[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    int e = -1, e_start = 0, e_end = 0, e_len = 0;
    float* st = nullptr;
    for (int t = t0; t < t1; ++t) {
        if (e < 0 || t >= e_end) {
            e = entry_of_row(q_start, q_len, E, t);
            if (e < 0) continue;
            e_start = q_start[e];
            e_len = q_len[e];
            e_end = e_start + e_len;
            st = taps > 1 ? state + (long long)slots[e] * slot_stride : nullptr;
            const int rel = t - e_start;
#pragma unroll
            for (int b = 1; b < MAX_TAPS; ++b) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (b < taps) v = rel - b >= 0 ? rows_at4(in, t - b, c) : *reinterpret_cast<const float4*>(st + (long long)(rel - b + taps - 1) * C + c);
                win[MAX_TAPS - 1 - b] = v;
            }
        }
        const float4 u = rows_at4(in, t, c);
        win[MAX_TAPS - 1] = u;
        if (out_copy != nullptr) store4<TOUT>(out_copy + (size_t)t * C + c, u);
        if (out_conv != nullptr) {
            float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
            if (taps > 0) {
#pragma unroll
                for (int i = 0; i < MAX_TAPS; ++i) {
                    y.x = fmaf(wr[0][i], win[i].x, y.x);
                    y.y = fmaf(wr[1][i], win[i].y, y.y);
                    y.z = fmaf(wr[2][i], win[i].z, y.z);
                    y.w = fmaf(wr[3][i], win[i].w, y.w);
                }
            }
            if (add_input) { y.x += u.x; y.y += u.y; y.z += u.z; y.w += u.w; }
            if (out_bias != nullptr) { y.x += ob.x; y.y += ob.y; y.z += ob.z; y.w += ob.w; }
            if (act == 1) {
                y.x = y.x / (1.f + expf(-y.x)); y.y = y.y / (1.f + expf(-y.y));
                y.z = y.z / (1.f + expf(-y.z)); y.w = y.w / (1.f + expf(-y.w));
            }
            store4<TOUT>(out_conv + (size_t)t * C + c, y);
        }
        if (taps > 1 && e_len == 1) state_push4(st, C, taps, c, u);
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i) win[i] = win[i + 1];
    }
}

__global__ void conv_state_update_kernel(RowsIn in, float* __restrict__ state, long long slot_stride,
                                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                                         const int* __restrict__ slots, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = q_len[e];
    if (c >= C || n <= 1) return;    // (an entry of one token was brought up to date by the kernel that convolved it)
    float* st = state + (long long)slots[e] * slot_stride;
    const int keep = taps - 1;
    float old[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) old[k] = k < keep ? st[(long long)k * C + c] : 0.f;
    const long long row0 = q_start[e];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) {
        if (k < keep) {
            const int rel = n - keep + k;   // place within the portion of the input that lands in row k
            float v;
            if (rel >= 0) v = rows_at(in, row0 + rel, c);
            else {
                // fewer new tokens than the state holds: the old rows move up (index n + k < keep)
                v = 0.f;
#pragma unroll
                for (int m = 0; m < MAX_TAPS; ++m)
                    if (m == n + k) v = old[m];
            }
            st[(long long)k * C + c] = v;
        }
    }
}

struct QkvArgs {
    RowsIn in;
    const float* w;       // [C][taps] or null when taps == 0
    float* state;
    long long slot_stride;
    const int* q_start;
    const int* q_len;
    const int* slots;
    const int* slot_map;  // [T]: page * page_size + offset of the token's cache entry, -1: none
    int E, C, taps;
    int nh, nkv, hd, hd_v;
    int use_norm;
    float eps;
    void* q_out;          // [T][nh * hd]
    void* pages;
    long long page_stride;
    int page_size, num_pages;
    int has_kv;
    int* status;
};

// a block a row; its warps take the heads in turn (query heads, then key heads, then value heads)
template <typename TOUT, bool VEC>
__global__ __launch_bounds__(256) void qkv_conv_norm_store_kernel(QkvArgs a) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int e = entry_of_row(a.q_start, a.q_len, a.E, t);
    if (e < 0) return;
    const int lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int warp = (threadIdx.x >> 5) + blockIdx.y * nwarps;     // the head this warp takes
    const int rel = t - a.q_start[e];
    float* st = a.state != nullptr ? a.state + (long long)a.slots[e] * a.slot_stride : nullptr;
    const bool push = a.taps > 1 && a.q_len[e] == 1;   // one token: the state is brought up to date here
    const int units = a.nh + (a.has_kv ? 2 * a.nkv : 0);
    long long slot = -1;
    if (a.has_kv) {
        slot = a.slot_map[t];
        if (slot >= (long long)a.num_pages * a.page_size) {
            if (threadIdx.x == 0 && a.status != nullptr) atomicOr(a.status, VCB_STATUS_BAD_PAGE);
            slot = -1;
        }
    }
    TOUT* q_out = reinterpret_cast<TOUT*>(a.q_out);
    TOUT* pages = reinterpret_cast<TOUT*>(a.pages);
    constexpr int PER = VCB_MAX_HEAD_DIM / 32;
    if (VEC) {
        // four neighbouring lanes of the head a thread: 16-byte loads, 8- or 16-byte stores
        constexpr int PER4 = VCB_MAX_HEAD_DIM / 128;
        const int u = warp;
        if (u >= units) return;
        int c0, n, kind;
        if (u < a.nh) { kind = 0; n = a.hd; c0 = u * a.hd; }
        else if (u < a.nh + a.nkv) { kind = 1; n = a.hd; c0 = a.nh * a.hd + (u - a.nh) * a.hd; }
        else { kind = 2; n = a.hd_v; c0 = (a.nh + a.nkv) * a.hd + (u - a.nh - a.nkv) * a.hd_v; }
        float4 y[PER4];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PER4; ++i) {
            const int d = 4 * (lane + 32 * i);
            y[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (d < n) {
                y[i] = a.taps > 0 ? conv_at4(a.in, a.w, st, a.C, a.taps, t, rel, c0 + d) : rows_at4(a.in, t, c0 + d);
                if (push) state_push4(st, a.C, a.taps, c0 + d, rows_at4(a.in, t, c0 + d));
                ss += y[i].x * y[i].x + y[i].y * y[i].y + y[i].z * y[i].z + y[i].w * y[i].w;
            }
        }
        float mul = 1.f;
        if (kind != 2 && a.use_norm) {
            ss = warp_sum(ss);
            mul = 1.f / sqrtf(ss / (float)n + a.eps);
        }
        TOUT* dst = nullptr;
        if (kind == 0) dst = q_out + (size_t)t * a.nh * a.hd + c0;
        else if (slot >= 0) {
            const long long page = slot / a.page_size, off = slot % a.page_size;
            const int kvh = kind == 1 ? u - a.nh : u - a.nh - a.nkv;
            dst = pages + page * a.page_stride +
                  (kind == 1 ? ((long long)kvh * a.page_size + off) * a.hd
                             : (long long)a.nkv * a.page_size * a.hd + ((long long)kvh * a.page_size + off) * a.hd_v);
        }
        if (dst != nullptr) {
#pragma unroll
            for (int i = 0; i < PER4; ++i) {
                const int d = 4 * (lane + 32 * i);
                if (d < n) store4<TOUT>(dst + d, make_float4(y[i].x * mul, y[i].y * mul, y[i].z * mul, y[i].w * mul));
            }
        }
        return;
    }
    for (int u = warp; u < units; u += nwarps * gridDim.y) {
        int c0, n, kind;   // kind 0: query, 1: key, 2: value
        if (u < a.nh) { kind = 0; n = a.hd; c0 = u * a.hd; }
        else if (u < a.nh + a.nkv) { kind = 1; n = a.hd; c0 = a.nh * a.hd + (u - a.nh) * a.hd; }
        else { kind = 2; n = a.hd_v; c0 = (a.nh + a.nkv) * a.hd + (u - a.nh - a.nkv) * a.hd_v; }
        float y[PER];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            y[i] = 0.f;
            if (d < n) {
                y[i] = a.taps > 0 ? conv_at(a.in, a.w, st, a.C, a.taps, t, rel, c0 + d) : rows_at(a.in, t, c0 + d);
                if (push) state_push(st, a.C, a.taps, c0 + d, rows_at(a.in, t, c0 + d));
                ss = fmaf(y[i], y[i], ss);
            }
        }
        float mul = 1.f;
        if (kind != 2 && a.use_norm) {
            ss = warp_sum(ss);
            mul = 1.f / sqrtf(ss / (float)n + a.eps);
        }
        if (kind == 0) {
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + 32 * i;
                if (d < n) q_out[(size_t)t * a.nh * a.hd + c0 + d] = from_f32<TOUT>(y[i] * mul);
            }
        } else if (slot >= 0) {
            const long long page = slot / a.page_size, off = slot % a.page_size;
            const int kvh = kind == 1 ? u - a.nh : u - a.nh - a.nkv;
            const long long base = page * a.page_stride +
                                   (kind == 1 ? ((long long)kvh * a.page_size + off) * a.hd
                                              : (long long)a.nkv * a.page_size * a.hd + ((long long)kvh * a.page_size + off) * a.hd_v);
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + 32 * i;
                if (d < n) pages[base + d] = from_f32<TOUT>(y[i] * mul);
            }
        }
    }
}

// x_t += w * n(y_t * sigmoid(g_t + b)); a block a row, the gated values kept in shared memory between the two passes
template <typename TOUT>
__global__ void gated_norm_add_kernel(float* __restrict__ resid, RowsIn y, RowsIn g, const float* __restrict__ w, float eps,
                                      const int* __restrict__ q_start, const int* __restrict__ q_len, int E, int H,
                                      TOUT* __restrict__ out_cast) {
    extern __shared__ float vals[];   // [H] then 33 floats for the block sum
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if (entry_of_row(q_start, q_len, E, t) < 0) return;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = rows_at(y, t, c);
        if (g.p != nullptr) v *= 1.f / (1.f + expf(-rows_at(g, t, c)));
        vals[c] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, vals + H);
    const float mul = 1.f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float x = resid[(size_t)t * H + c] + vals[c] * mul * w[c];
        resid[(size_t)t * H + c] = x;
        if (out_cast != nullptr) out_cast[(size_t)t * H + c] = from_f32<TOUT>(x);
    }
}

// the same with four channels a thread and everything a thread needs held in registers: every load of the row is
// asked for before the first result is needed
template <typename TOUT, int VPT>
__global__ __launch_bounds__(1024) void gated_norm_add_vec_kernel(float* __restrict__ resid, RowsIn y, RowsIn g,
                                                                  const float* __restrict__ w, float eps,
                                                                  const int* __restrict__ q_start, const int* __restrict__ q_len,
                                                                  int E, int H, TOUT* __restrict__ out_cast) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if (entry_of_row(q_start, q_len, E, t) < 0) return;
    const int nv = H >> 2;
    float4 v[VPT], r[VPT], gs[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nv) {
            r[i] = *reinterpret_cast<const float4*>(resid + (size_t)t * H + 4 * idx);
            v[i] = rows_at4(y, t, 4 * idx);
            if (g.p != nullptr) gs[i] = rows_at4(g, t, 4 * idx);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nv) {
            if (g.p != nullptr) {
                v[i].x *= 1.f / (1.f + expf(-gs[i].x)); v[i].y *= 1.f / (1.f + expf(-gs[i].y));
                v[i].z *= 1.f / (1.f + expf(-gs[i].z)); v[i].w *= 1.f / (1.f + expf(-gs[i].w));
            }
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float mul = 1.f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nv) {
            const float4 ww = *reinterpret_cast<const float4*>(w + 4 * idx);
            float4 x = r[i];
            x.x += v[i].x * mul * ww.x; x.y += v[i].y * mul * ww.y; x.z += v[i].z * mul * ww.z; x.w += v[i].w * mul * ww.w;
            *reinterpret_cast<float4*>(resid + (size_t)t * H + 4 * idx) = x;
            if (out_cast != nullptr) store4<TOUT>(out_cast + (size_t)t * H + 4 * idx, x);
        }
    }
}

template <typename TOUT>
__global__ void bias_act_vec_kernel(RowsIn in, TOUT* __restrict__ out, int T, int C4, int kind) {
    pdl_trigger();
    pdl_wait();
    // a row a block in turn, four channels a thread: no division on the way to an address
    for (int t = blockIdx.y; t < T; t += gridDim.y)
    for (int c4 = blockIdx.x * blockDim.x + threadIdx.x; c4 < C4; c4 += gridDim.x * blockDim.x) {
        const int c = 4 * c4;
        float4 z = rows_at4(in, t, c);
        float* f = reinterpret_cast<float*>(&z);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float x = f[k];
            if (kind == 0) f[k] = 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
            else if (kind == 1) f[k] = 0.5f * x * (1.f + tanhf(0.79788456080286535588f * (x + 0.044715f * x * x * x)));
            else if (kind == 2) f[k] = x / (1.f + expf(-x));
            else if (kind == 3) { const float r = fmaxf(x, 0.f); f[k] = r * r; }
        }
        store4<TOUT>(out + (size_t)t * (4 * (size_t)C4) + c, z);
    }
}

template <typename TOUT>
__global__ void bias_act_kernel(RowsIn in, TOUT* __restrict__ out, long long total, int C, int kind) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / C;
        const int c = (int)(i % C);
        const float z = rows_at(in, t, c);
        float r;
        if (kind == 0) r = 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
        else if (kind == 1) r = 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
        else if (kind == 2) r = z / (1.f + expf(-z));
        else if (kind == 3) { const float p = fmaxf(z, 0.f); r = p * p; }
        else r = z;
        out[i] = from_f32<TOUT>(r);
    }
}

}  // namespace

VCB_API int vcb_embed_sinusoid(const void* table, int table_dtype, const int* ids, const int* positions,
                               const float* inv_freq, float* out, int T, int H, int V, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    launch_pdl(embed_sinusoid_kernel, dim3(T), dim3(256), 0, stream, table, table_dtype, ids, positions, inv_freq, out, H, V, status);
    VCB_CHECK_LAUNCH("embed_sinusoid");
    return 0;
}

// in: [S][T][ld] 32-bit (+ bias); out_conv = conv(in) (+ in with add_input), out_copy = in, both [T][C] of out_dtype,
// either may be null.  taps 0: no convolution (out_conv = in with add_input, else zeros).  state [slots][taps-1][C]:
// read, and for entries of one token brought up to date as well (entries of more need vcb_conv_state_update afterwards).
// out_bias [C] (or null) is added to the convolution's result, then act (0: none, 1: SiLU) is applied to it.
VCB_API int vcb_causal_conv(const float* in, int S, long long s_stride, long long ld, const float* bias, const float* w,
                            float* state, long long slot_stride, const int* q_start, const int* q_len,
                            const int* slots, int E, int T, int C, int taps, int add_input, void* out_conv,
                            void* out_copy, int out_dtype, const float* out_bias, int act, cudaStream_t stream) {
    if (T == 0 || C == 0) return 0;
    VCB_CHECK_ARG(taps >= 0 && taps <= MAX_TAPS, "causal_conv: %d taps (0 to %d)", taps, MAX_TAPS);
    VCB_CHECK_ARG(taps < 2 || state != nullptr, "causal_conv: a convolution over %d tokens needs the requests' state", taps);
    VCB_CHECK_ARG(T <= 65535, "causal_conv: %d rows in one step (at most 65535)", T);
    RowsIn r{in, S < 1 ? 1 : S, s_stride, ld, bias};
    VCB_CHECK_ARG(act == 0 || act == 1, "causal_conv: unknown activation %d", act);
    const bool vec = C % 4 == 0 && rows_vec_ok(r) && (uintptr_t)out_conv % 16 == 0 && (uintptr_t)out_copy % 16 == 0 &&
                     (uintptr_t)out_bias % 16 == 0 &&
                     (state == nullptr || ((uintptr_t)state % 16 == 0 && slot_stride % 4 == 0));
    if (vec && T >= 512) {
        // many rows: runs of 16 rows a thread, the inputs fetched once
        constexpr int RUN = 16;
        const dim3 gridr((C / 4 + 127) / 128, (T + RUN - 1) / RUN), blockr(128);
        if (out_dtype == VCB_F32)
            launch_pdl(causal_conv_run_kernel<float, RUN>, gridr, blockr, 0, stream, r, w, state, slot_stride, q_start, q_len, slots, E, T,
                       C, taps, add_input, (float*)out_conv, (float*)out_copy, out_bias, act);
        else
            launch_pdl(causal_conv_run_kernel<__nv_bfloat16, RUN>, gridr, blockr, 0, stream, r, w, state, slot_stride, q_start, q_len,
                       slots, E, T, C, taps, add_input, (__nv_bfloat16*)out_conv, (__nv_bfloat16*)out_copy, out_bias, act);
        VCB_CHECK_LAUNCH("causal_conv");
        return 0;
    }
    if (vec) {
        const dim3 grid4((C / 4 + 127) / 128, T), block4(128);
        if (out_dtype == VCB_F32)
            launch_pdl(causal_conv_vec_kernel<float>, grid4, block4, 0, stream, r, w, state, slot_stride, q_start, q_len, slots, E, T,
                       C, taps, add_input, (float*)out_conv, (float*)out_copy, out_bias, act);
        else
            launch_pdl(causal_conv_vec_kernel<__nv_bfloat16>, grid4, block4, 0, stream, r, w, state, slot_stride, q_start, q_len,
                       slots, E, T, C, taps, add_input, (__nv_bfloat16*)out_conv, (__nv_bfloat16*)out_copy, out_bias, act);
        VCB_CHECK_LAUNCH("causal_conv");
        return 0;
    }
    const dim3 grid((C + 255) / 256, T), block(256);
    if (out_dtype == VCB_F32)
        launch_pdl(causal_conv_kernel<float>, grid, block, 0, stream, r, w, state, slot_stride, q_start, q_len, slots, E, T, C,
                   taps, add_input, (float*)out_conv, (float*)out_copy, out_bias, act);
    else
        launch_pdl(causal_conv_kernel<__nv_bfloat16>, grid, block, 0, stream, r, w, state, slot_stride, q_start, q_len, slots, E,
                   T, C, taps, add_input, (__nv_bfloat16*)out_conv, (__nv_bfloat16*)out_copy, out_bias, act);
    VCB_CHECK_LAUNCH("causal_conv");
    return 0;
}

VCB_API int vcb_conv_state_update(const float* in, int S, long long s_stride, long long ld, const float* bias, float* state,
                                  long long slot_stride, const int* q_start, const int* q_len, const int* slots, int E,
                                  int C, int taps, cudaStream_t stream) {
    if (E == 0 || C == 0 || taps < 2) return 0;
    VCB_CHECK_ARG(taps <= MAX_TAPS, "conv_state_update: %d taps (at most %d)", taps, MAX_TAPS);
    VCB_CHECK_ARG(E <= 65535, "conv_state_update: %d entries in one step (at most 65535)", E);
    RowsIn r{in, S < 1 ? 1 : S, s_stride, ld, bias};
    launch_pdl(conv_state_update_kernel, dim3((C + 255) / 256, E), dim3(256), 0, stream, r, state, slot_stride, q_start, q_len,
               slots, C, taps);
    VCB_CHECK_LAUNCH("conv_state_update");
    return 0;
}

VCB_API int vcb_qkv_conv_norm_store(const float* in, int S, long long s_stride, long long ld, const float* bias,
                                    const float* w, float* state, long long slot_stride, const int* q_start,
                                    const int* q_len, const int* slots, const int* slot_map, int E, int T, int taps, int nh,
                                    int nkv, int hd, int hd_v, int use_norm, float eps, void* q_out, void* pages,
                                    long long page_stride, int page_size, int num_pages, int has_kv, int out_dtype,
                                    int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(taps >= 0 && taps <= MAX_TAPS, "qkv_conv_norm_store: %d taps (0 to %d)", taps, MAX_TAPS);
    VCB_CHECK_ARG(taps < 2 || state != nullptr, "qkv_conv_norm_store: a convolution over %d tokens needs the requests' state", taps);
    VCB_CHECK_ARG(hd >= 1 && hd <= VCB_MAX_HEAD_DIM && hd_v >= 1 && hd_v <= VCB_MAX_HEAD_DIM,
                  "qkv_conv_norm_store: head sizes %d and %d must lie in [1, %d]", hd, hd_v, VCB_MAX_HEAD_DIM);
    QkvArgs a{};
    a.in = RowsIn{in, S < 1 ? 1 : S, s_stride, ld, bias};
    a.w = w; a.state = state; a.slot_stride = slot_stride;
    a.q_start = q_start; a.q_len = q_len; a.slots = slots; a.slot_map = slot_map;
    a.E = E; a.C = nh * hd + (has_kv ? nkv * (hd + hd_v) : 0); a.taps = taps;
    a.nh = nh; a.nkv = nkv; a.hd = hd; a.hd_v = hd_v; a.use_norm = use_norm; a.eps = eps;
    a.q_out = q_out; a.pages = pages; a.page_stride = page_stride; a.page_size = page_size; a.num_pages = num_pages;
    a.has_kv = has_kv; a.status = status;
    const int units = nh + (has_kv ? 2 * nkv : 0);
    const int warps = units < 4 ? units : 4;
    const dim3 grid(T, (units + warps - 1) / warps), block(32 * warps);
    VCB_CHECK_ARG(grid.y <= 65535, "qkv_conv_norm_store: %d heads", units);
    const size_t esz = out_dtype == VCB_F32 ? 4 : 2;
    const bool vec = hd % 4 == 0 && hd_v % 4 == 0 && rows_vec_ok(a.in) && (state == nullptr || ((uintptr_t)state % 16 == 0 && slot_stride % 4 == 0)) &&
                     (uintptr_t)q_out % 16 == 0 && (!has_kv || ((uintptr_t)pages % 16 == 0 && (page_stride * esz) % 16 == 0 &&
                                                               ((long long)nkv * page_size * hd * esz) % 16 == 0));
    if (out_dtype == VCB_F32) {
        if (vec) launch_pdl(qkv_conv_norm_store_kernel<float, true>, grid, block, 0, stream, a);
        else launch_pdl(qkv_conv_norm_store_kernel<float, false>, grid, block, 0, stream, a);
    } else {
        if (vec) launch_pdl(qkv_conv_norm_store_kernel<__nv_bfloat16, true>, grid, block, 0, stream, a);
        else launch_pdl(qkv_conv_norm_store_kernel<__nv_bfloat16, false>, grid, block, 0, stream, a);
    }
    VCB_CHECK_LAUNCH("qkv_conv_norm_store");
    return 0;
}

// y: the sublayer's result [Sy][T][ldy]; g: the gate's sums [Sg][T][ldg] with bias gb, or null: no gate.
// out_cast (or null): the updated rows once more, in out_dtype.
VCB_API int vcb_gated_norm_add(float* resid, const float* y, int Sy, long long y_stride, long long ldy, const float* g, int Sg,
                               long long g_stride, long long ldg, const float* gb, const float* w, float eps,
                               const int* q_start, const int* q_len, int E, int T, int H, void* out_cast, int out_dtype,
                               cudaStream_t stream) {
    if (T == 0) return 0;
    RowsIn ry{y, Sy < 1 ? 1 : Sy, y_stride, ldy, nullptr};
    RowsIn rg{g, Sg < 1 ? 1 : Sg, g_stride, ldg, gb};
    if (H % 4 == 0 && H / 4 <= 4096 && rows_vec_ok(ry) && rows_vec_ok(rg) && (uintptr_t)resid % 16 == 0 && (uintptr_t)w % 16 == 0 &&
        (uintptr_t)out_cast % 16 == 0) {
        const int nv = H / 4;
        const int vpt = nv <= 1024 ? 1 : (nv <= 2048 ? 2 : 4);
        const int threads4 = ((nv + vpt - 1) / vpt + 31) / 32 * 32;
#define VCB_GNA(TOUT, V) launch_pdl(gated_norm_add_vec_kernel<TOUT, V>, dim3(T), dim3(threads4), 0, stream, resid, ry, rg, w, eps, q_start, q_len, E, H, (TOUT*)out_cast)
        if (out_dtype == VCB_F32) { if (vpt == 1) VCB_GNA(float, 1); else if (vpt == 2) VCB_GNA(float, 2); else VCB_GNA(float, 4); }
        else { if (vpt == 1) VCB_GNA(__nv_bfloat16, 1); else if (vpt == 2) VCB_GNA(__nv_bfloat16, 2); else VCB_GNA(__nv_bfloat16, 4); }
#undef VCB_GNA
        VCB_CHECK_LAUNCH("gated_norm_add");
        return 0;
    }
    const size_t smem = ((size_t)H + 64) * sizeof(float);
    const int threads = H >= 1024 ? 1024 : (H >= 512 ? 512 : 256);
    if (out_dtype == VCB_F32) {
        auto kern = gated_norm_add_kernel<float>;
        if (smem > 48 * 1024) VCB_CHECK_ARG(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
                                            "gated_norm_add: %zu bytes of shared memory refused", smem);
        launch_pdl(kern, dim3(T), dim3(threads), smem, stream, resid, ry, rg, w, eps, q_start, q_len, E, H, (float*)out_cast);
    } else {
        auto kern = gated_norm_add_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) VCB_CHECK_ARG(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
                                            "gated_norm_add: %zu bytes of shared memory refused", smem);
        launch_pdl(kern, dim3(T), dim3(threads), smem, stream, resid, ry, rg, w, eps, q_start, q_len, E, H, (__nv_bfloat16*)out_cast);
    }
    VCB_CHECK_LAUNCH("gated_norm_add");
    return 0;
}

// kind 0: GELU with erf, 1: GELU with tanh, 2: SiLU, 3: the square of ReLU, 4: none (the sums, plus bias, in out_dtype)
VCB_API int vcb_bias_act(const float* in, int S, long long s_stride, long long ld, const float* bias, void* out, int out_dtype,
                         int T, int C, int kind, cudaStream_t stream) {
    if (T == 0 || C == 0) return 0;
    VCB_CHECK_ARG(kind >= 0 && kind <= 4, "bias_act: unknown activation %d", kind);
    RowsIn r{in, S < 1 ? 1 : S, s_stride, ld, bias};
    const long long total = (long long)T * C;
    if (C % 4 == 0 && rows_vec_ok(r) && (uintptr_t)out % 16 == 0) {
        const int bx = (C / 4 + 255) / 256 < 64 ? (C / 4 + 255) / 256 : 64;
        const dim3 grid4(bx, T < 65535 ? T : 65535);
        if (out_dtype == VCB_F32) launch_pdl(bias_act_vec_kernel<float>, grid4, dim3(256), 0, stream, r, (float*)out, T, C / 4, kind);
        else launch_pdl(bias_act_vec_kernel<__nv_bfloat16>, grid4, dim3(256), 0, stream, r, (__nv_bfloat16*)out, T, C / 4, kind);
        VCB_CHECK_LAUNCH("bias_act");
        return 0;
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (out_dtype == VCB_F32) launch_pdl(bias_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, r, (float*)out, total, C, kind);
    else launch_pdl(bias_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, r, (__nv_bfloat16*)out, total, C, kind);
    VCB_CHECK_LAUNCH("bias_act");
    return 0;
}
