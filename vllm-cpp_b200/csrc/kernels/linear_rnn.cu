// Recurrent mixers whose state is a matrix per head, S [d][dv] in 32-bit, carried from token to token in the request's slot:
//
//  * the gated delta rule    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                            q, k: the head's rows of a convolved buffer, made unit vectors here (x / sqrt(sum x^2 + 1e-6)),
//                            q times d^(-1/2); beta = sigmoid(b); g = exp(-rate_h softplus(a + dt_bias_h))
//  * the gated linear form   S <- diag(f) S + (1 - f) v^T;  o = S^T q
//                            q = silu(.), f = low + (1 - low) sigmoid(. + bias), all from one row of 32-bit sums
//  * the decayed form        S <- diag(f) S + k v^T;  o = S^T q
//                            q times d^(-1/2), k, v from one row of 32-bit sums; f = sigmoid(z + bias)^(1/tau) per state row,
//                            z the sums of a second (low-rank) projection: exp(-softplus(-(z + bias)) / tau) in 32-bit
//  * retention               S <- decay_h S + k v^T;  o = S^T q
//                            one fixed decay per head; the first `rot` lanes of q and k turned by position * freq[i]
//                            (pairs in halves or interleaved), k then times d^(-1/2)
//  * head_norm_gate          every head of o divided by its root mean square, times a gain shared by the heads, times
//                            silu(gate) where there is a gate
//
// One token after the other is the only order the recurrences allow.  A block owns (entry, head, a tile of value columns).
// Its first WALKERS threads walk the tokens: a thread keeps R rows of two neighbouring columns in registers, in pieces of
// four rows dealt round to the L neighbouring lanes that share the columns, so a token's q and k come as 16-byte words
// from shared memory (each serving both columns) and the state as 16-byte words from its slot; the arithmetic runs on
// pairs of 32-bit lanes (fma.rn.f32x2).  The lanes' partial sums meet in shuffles; a token's read-out is reduced in the
// same rounds as the next token's S^T k, so one set of rounds a token is on the critical path.  Its other STAGERS threads
// meanwhile fetch the next TB tokens' inputs into the other half of a double buffer in shared memory (gates, decays,
// unit norms done there), so the walk never waits for memory.  A step of decoded tokens runs blocks of WALKERS threads
// that stage and then walk.  The order of every sum depends on d only, never on how a prompt was cut or on which of the
// two forms ran: a cut changes nothing but the place of a barrier.
#include "common.cuh"

namespace {

constexpr int WALKERS = 256;    // threads that walk the tokens
constexpr int STAGERS = 256;    // threads that stage the tokens after these
constexpr int THREADS = WALKERS + STAGERS;
constexpr int U = 8;            // loads a stager has in flight per kind

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

template <bool ONE>
__device__ __forceinline__ float sums_at(const Rows& in, long long t, int c) {
    return ONE ? in.p[t * in.ld + c] : rows_at(in, t, c);
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
// two 32-bit lanes in one 64-bit register; fma.rn.f32x2 and mul.rn.f32x2 are an IEEE operation on each lane
__device__ __forceinline__ uint64_t pair_f32(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpair_f32(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_pair(uint64_t x, uint64_t y, uint64_t z) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(x), "l"(y), "l"(z));
    return d;
}
__device__ __forceinline__ uint64_t mul_pair(uint64_t x, uint64_t y) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(x), "l"(y));
    return d;
}
__device__ __forceinline__ void group_barrier(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

enum { MODE_DELTA = 0, MODE_GATED = 1, MODE_DECAYED = 2, MODE_RETAIN = 3 };

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
    float* state;           // [slots][H][dv][d]
    long long state_stride;
    const int* q_start;
    const int* q_len;
    const int* slots;
    float* out;             // [T][H * dv]
    int H, G, d, dv, L;     // G heads of q and k (MODE_DELTA; head h reads h / (H / G))
    int TB, dp_shift, ct_shift;     // tokens staged at a time; log2(L * R); log2(value columns a block owns)
    Rows z;                 // MODE_DECAYED: the decay's sums [T][H * d]; f_bias is their bias
    float inv_tau;          // MODE_DECAYED: 1 / tau
    const float* decay;     // MODE_RETAIN: [H]
    const int* ctx_len;     // MODE_RETAIN: an entry's tokens end at this position
    const float* freq;      // MODE_RETAIN: [rot / 2]
    int rot, interleaved;   // MODE_RETAIN: lanes of q and k that turn, and how they pair
};

struct Stage {              // one half of the double buffer
    float* q;               // [TB][L * R]
    float* k;               // [TB][L * R]   (MODE_GATED: the forget gate)
    float* f;               // [TB][L * R]   (MODE_DECAYED only: the decay of every state row)
    float* v;               // [TB][CT]
    float* g;               // [TB]
    float* b;               // [TB]
};

// the inputs of tokens t_first .. t_first + nb - 1 of (entry, head h, value columns from c0) into `s`; all STAGERS threads.
// A thread fetches one q/k row (two where a token has more rows than there are stagers) of every tpr-th token, so its
// addresses differ by a multiple of the row stride only; the loads of a round are all in flight before the first is used.
// (ONE: the sums are one slice, so a load has no add behind it.)
template <int MODE, bool ONE, int R>
__device__ __forceinline__ void stage_tokens(const RnnArgs& a, const Stage& s, int ltid, int h, int hk, long long t_first, int nb,
                                             int c0, int pos_first) {
    const int d = a.d, dv = a.dv, DP = 1 << a.dp_shift, DPP = DP, CT = 1 << a.ct_shift, TB = a.TB;
    const int ldx = (int)a.ldx, ldu = (int)a.u.ld;
    // v, beta and the decay first: their loads fly while q and k are fetched
    const float* vp = MODE == MODE_DELTA ? a.x + t_first * a.ldx + a.v_col + h * dv + c0 : a.u.p + t_first * a.u.ld + a.v_col + h * dv + c0;
    const int ldv = MODE == MODE_DELTA ? ldx : ldu;
    auto v_at = [&](int idx) {
        const int tt = idx >> a.ct_shift, c = idx & (CT - 1);
        if (idx >= TB * CT || tt >= nb || c0 + c >= dv) return 0.f;
        return (MODE == MODE_DELTA || ONE) ? vp[tt * ldv + c] : rows_at(a.u, t_first + tt, a.v_col + h * dv + c0 + c);
    };
    float vv[2];
#pragma unroll
    for (int w = 0; w < 2; ++w) vv[w] = v_at(ltid + w * STAGERS);
    float braw = 0.f, araw = 0.f;
    if (MODE == MODE_DELTA && ltid < nb) {
        braw = sums_at<ONE>(a.u, t_first + ltid, a.b_col + h);
        araw = sums_at<ONE>(a.u, t_first + ltid, a.a_col + h);
    }
    const int tpr = max(1, STAGERS >> a.dp_shift), tt0 = ltid >> a.dp_shift;
    for (int i = ltid & (DP - 1); i < DP; i += STAGERS) {
        const bool in = i < d;
        const int pi = i;
        const float *qp, *kp;
        float low = 0.f, fb = 0.f;
        if (MODE == MODE_DELTA) {
            qp = a.x + t_first * a.ldx + a.q_col + hk * d + i;
            kp = a.x + t_first * a.ldx + a.k_col + hk * d + i;
        } else {
            qp = a.u.p + t_first * a.u.ld + a.q_col + h * d + i;
            kp = a.u.p + t_first * a.u.ld + a.k_col + h * d + i;
            if (in) {
                low = a.lower[h * d + i];
                fb = a.f_bias[h * d + i];
            }
        }
        if (MODE == MODE_DECAYED && in) fb = a.f_bias[h * d + i];
        const float dscale = rsqrtf((float)d);
        const int ldq = MODE == MODE_DELTA ? ldx : ldu;
        for (int tb = tt0; tb < TB; tb += U * tpr) {
            float qv[U], kv[U], fv[MODE == MODE_DECAYED ? U : 1];
#pragma unroll
            for (int w = 0; w < U; ++w) {
                const int tt = tb + w * tpr;
                qv[w] = 0.f;
                kv[w] = 0.f;
                if constexpr (MODE == MODE_DECAYED) fv[w] = 0.f;
                if (in && tt < nb) {
                    if (MODE == MODE_DELTA || ONE) {
                        qv[w] = qp[tt * ldq];
                        kv[w] = kp[tt * ldq];
                    } else {
                        qv[w] = rows_at(a.u, t_first + tt, a.q_col + h * d + i);
                        kv[w] = rows_at(a.u, t_first + tt, a.k_col + h * d + i);
                    }
                    if constexpr (MODE == MODE_DECAYED) fv[w] = rows_at(a.z, t_first + tt, h * d + i);
                }
            }
#pragma unroll
            for (int w = 0; w < U; ++w) {
                const int tt = tb + w * tpr;
                if (tt < TB) {
                    if (MODE == MODE_GATED && in && tt < nb) {
                        qv[w] = silu_f(qv[w]);
                        kv[w] = low + (1.f - low) * sigmoid_f(kv[w] + fb);
                    }
                    if constexpr (MODE == MODE_DECAYED) {
                        qv[w] *= dscale;
                        // sigmoid(x)^(1/tau) = exp(-softplus(-x) / tau); rows beyond d keep a zero state whatever they hold
                        s.f[tt * DPP + pi] = in && tt < nb ? expf(-softplus_f(-(fv[w] + fb)) * a.inv_tau) : 0.f;
                    }
                    if (MODE == MODE_RETAIN && i >= a.rot) kv[w] *= dscale;     // (the turning lanes after their turn)
                    s.q[tt * DPP + pi] = qv[w];
                    s.k[tt * DPP + pi] = kv[w];
                }
            }
        }
    }
#pragma unroll
    for (int w = 0; w < 2; ++w)
        if (ltid + w * STAGERS < TB * CT) s.v[ltid + w * STAGERS] = vv[w];
    for (int idx = ltid + 2 * STAGERS; idx < TB * CT; idx += STAGERS) s.v[idx] = v_at(idx);
    if (MODE == MODE_DELTA) {
        if (ltid < nb) {
            s.b[ltid] = sigmoid_f(braw);
            s.g[ltid] = expf(-a.rate[h] * softplus_f(araw + a.dt_bias[h]));
        }
        group_barrier(1, STAGERS);
        // q and k as unit vectors (a warp a token), q times d^(-1/2)
        const int lane = ltid & 31, warp = ltid >> 5;
        const float qscale = rsqrtf((float)d);
        for (int tt = warp; tt < nb; tt += STAGERS / 32) {
            float* q = s.q + tt * DPP;
            float* k = s.k + tt * DPP;
            float sq = 0.f, sk = 0.f;
            for (int i = lane; i < d; i += 32) {
                const int pi = i;
                sq = fmaf(q[pi], q[pi], sq);
                sk = fmaf(k[pi], k[pi], sk);
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            const float rq = rsqrtf(sq + 1e-6f) * qscale, rk = rsqrtf(sk + 1e-6f);
            for (int i = lane; i < d; i += 32) {
                const int pi = i;
                q[pi] *= rq;
                k[pi] *= rk;
            }
        }
    }
    if (MODE == MODE_RETAIN && a.rot > 0) {
        group_barrier(1, STAGERS);
        // q and k turned by the token's position, a thread a pair of lanes; k then times d^(-1/2)
        const int hr = a.rot >> 1;
        const float kscale = rsqrtf((float)d);
        for (int idx = ltid; idx < nb * hr; idx += STAGERS) {
            const int tt = idx / hr, i = idx % hr;
            const int la = a.interleaved ? 2 * i : i, lb = a.interleaved ? 2 * i + 1 : i + hr;
            float sn, cs;
            sincosf((float)(pos_first + tt) * a.freq[i], &sn, &cs);
            float* q = s.q + tt * DPP;
            float* k = s.k + tt * DPP;
            const float qa = q[la], qb = q[lb], ka = k[la], kb = k[lb];
            q[la] = qa * cs - qb * sn;
            q[lb] = qb * cs + qa * sn;
            k[la] = (ka * cs - kb * sn) * kscale;
            k[lb] = (kb * cs + ka * sn) * kscale;
        }
    }
}

// SPLIT: 512 threads, stagers beside walkers (long portions).  Otherwise 256 threads that stage and then walk, several blocks
// an SM: a step of decoded tokens is many short blocks, which hide one another's waits.  R: state rows a thread keeps of
// each of its C (one or two) columns: one column a thread where that still fills the GPU's SMs once, else two, which
// halves the shared-memory reads a column.
template <int MODE, bool SPLIT, int R, int C>
__global__ __launch_bounds__(SPLIT ? THREADS : WALKERS, SPLIT ? 1 : 2) void matrix_rnn_kernel(RnnArgs a) {
    extern __shared__ __align__(16) float sm[];
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.z, h = blockIdx.y;
    const int n = a.q_len[e];
    if (n <= 0) return;
    const int L = a.L, CT = 1 << a.ct_shift, DPP = L * R, TB = a.TB;
    const int d = a.d, dv = a.dv;
    constexpr int NQK = MODE == MODE_DECAYED ? 3 : 2;
    const int half = NQK * TB * DPP + TB * CT + 2 * TB;       // (a multiple of four lanes)
    auto stage_at = [&](int which) {
        Stage s;
        s.q = sm + which * half;
        s.k = s.q + TB * DPP;
        s.f = s.k + TB * DPP;
        s.v = s.q + NQK * TB * DPP;
        s.g = s.v + TB * CT;
        s.b = s.g + TB;
        return s;
    };
    float* o_s = sm + 2 * half;         // [TB][CT]
    const int tid = threadIdx.x;
    const bool walker = !SPLIT || tid < WALKERS;
    const bool stager = !SPLIT || tid >= WALKERS;
    const int ltid = SPLIT ? tid - WALKERS : tid;
    const int kl = tid & (L - 1), cg = (tid & (WALKERS - 1)) / L;       // this thread's columns: c0 + C cg, and the next
    const int c0 = blockIdx.x * CT;
    const long long t0 = a.q_start[e];
    const int hk = MODE == MODE_DELTA ? h / (a.H / a.G) : h;
    const bool one = a.u.S == 1 && (MODE != MODE_DECAYED || a.z.S == 1);
    const int pos0 = MODE == MODE_RETAIN ? a.ctx_len[e] - n : 0;       // position of the entry's first token
    float* st = a.state + (size_t)a.slots[e] * a.state_stride + (size_t)h * d * dv;     // [dv][d]: a column's rows in a run
    // this thread's rows: the pieces of four 4 (kl + L m) .. + 3, m < R / 4, so that the L threads of a column read
    // neighbouring 16-byte words of q, k and the state.  Pairs of rows in a 64-bit register: the multiply-adds run on pairs.
    uint64_t S[C][R / 2];
    const bool vec = (d & 3) == 0 && (reinterpret_cast<uintptr_t>(st) & 15) == 0;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int j = c0 + cg * C + c;
        const bool in = walker && j < dv;
#pragma unroll
        for (int m = 0; m < R / 4; ++m) {
            const int i = 4 * (kl + L * m);
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (in && i < d) {
                const float* src = st + (size_t)j * d + i;
                if (vec) t = *reinterpret_cast<const float4*>(src);
                else {
                    t.x = src[0];
                    if (i + 1 < d) t.y = src[1];
                    if (i + 2 < d) t.z = src[2];
                    if (i + 3 < d) t.w = src[3];
                }
            }
            S[c][2 * m] = pair_f32(t.x, t.y);
            S[c][2 * m + 1] = pair_f32(t.z, t.w);
        }
    }
    const int batches = (n + TB - 1) / TB;
    if (stager) {
        if (one) stage_tokens<MODE, true, R>(a, stage_at(0), ltid, h, hk, t0, min(TB, n), c0, pos0);
        else stage_tokens<MODE, false, R>(a, stage_at(0), ltid, h, hk, t0, min(TB, n), c0, pos0);
    }
    __syncthreads();
    for (int b = 0; b < batches; ++b) {
        const int b0 = b * TB;
        const int nb = min(TB, n - b0);
        if (walker) {
            const Stage s = stage_at(b & 1);
            const ulonglong2* q4 = reinterpret_cast<const ulonglong2*>(s.q) + kl;
            const ulonglong2* k4 = reinterpret_cast<const ulonglong2*>(s.k) + kl;
            const ulonglong2* f4 = reinterpret_cast<const ulonglong2*>(s.f) + kl;
            const float* vcol = s.v + cg * C;
            const int step4 = DPP / 4;
            const bool odd = kl & 1;
            float o_prev[C];
#pragma unroll
            for (int c = 0; c < C; ++c) o_prev[c] = 0.f;
            // The read-out of one token is reduced in the same rounds as the next token's S^T k (`with_p`).  With two
            // columns the lanes first swap a column of the read-out each, then add up the one they kept: lanes 0 and 1 of
            // the L end with the sums of the first and the second column.  p is summed to every lane.
            auto reduce = [&](int tt_of, bool with_p, float* p) {
                if (L > 1) {
                    float keep;
                    if (C == 2) keep = (odd ? o_prev[C - 1] : o_prev[0]) + __shfl_xor_sync(0xffffffffu, odd ? o_prev[0] : o_prev[C - 1], 1);
                    else keep = o_prev[0] + __shfl_xor_sync(0xffffffffu, o_prev[0], 1);
                    if (with_p) {
#pragma unroll
                        for (int c = 0; c < C; ++c) p[c] += __shfl_xor_sync(0xffffffffu, p[c], 1);
                    }
                    for (int off = 2; off < L; off <<= 1) {
                        keep += __shfl_xor_sync(0xffffffffu, keep, off);
                        if (with_p) {
#pragma unroll
                            for (int c = 0; c < C; ++c) p[c] += __shfl_xor_sync(0xffffffffu, p[c], off);
                        }
                    }
                    if (tt_of >= 0 && kl < C) o_s[tt_of * CT + cg * C + kl] = keep;
                } else if (tt_of >= 0) {
#pragma unroll
                    for (int c = 0; c < C; ++c) o_s[tt_of * CT + cg * C + c] = o_prev[c];
                }
            };
            // a token's k (then q) is fetched as soon as the token before has used its own for the last time, so the
            // shared-memory reads run beside the arithmetic
            uint64_t kr[R / 2], qr[R / 2], fr[MODE == MODE_DECAYED ? R / 2 : 1];
            auto fetch = [&](uint64_t* dst, const ulonglong2* src, int tt_of) {
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    const ulonglong2 t = src[tt_of * step4 + L * r];
                    dst[2 * r] = t.x;
                    dst[2 * r + 1] = t.y;
                }
            };
            fetch(kr, k4, 0);
            fetch(qr, q4, 0);
            if constexpr (MODE == MODE_DECAYED) fetch(fr, f4, 0);
            const float head_decay = MODE == MODE_RETAIN ? a.decay[h] : 0.f;
            for (int tt = 0; tt < nb; ++tt) {
                const int next = min(tt + 1, nb - 1);
                float v[C];
#pragma unroll
                for (int c = 0; c < C; ++c) v[c] = vcol[tt * CT + c];
                uint64_t o2[C];      // (sum over even rows, sum over odd rows)
#pragma unroll
                for (int c = 0; c < C; ++c) o2[c] = 0ull;
                if constexpr (MODE == MODE_DELTA) {
                    const float g = s.g[tt], beta = s.b[tt];
                    const uint64_t gg = pair_f32(g, g);
                    uint64_t p2[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) p2[c] = 0ull;
#pragma unroll
                    for (int m = 0; m < R / 2; ++m) {
#pragma unroll
                        for (int c = 0; c < C; ++c) p2[c] = fma_pair(S[c][m], kr[m], p2[c]);
                    }
                    float p[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        float even, oddp;
                        unpair_f32(p2[c], even, oddp);
                        p[c] = even + oddp;
                    }
                    reduce(tt - 1, true, p);
                    uint64_t w[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        const float wc = beta * (v[c] - g * p[c]);
                        w[c] = pair_f32(wc, wc);
                    }
#pragma unroll
                    for (int m = 0; m < R / 2; ++m) {
#pragma unroll
                        for (int c = 0; c < C; ++c) S[c][m] = fma_pair(kr[m], w[c], mul_pair(gg, S[c][m]));
                    }
                } else if constexpr (MODE == MODE_DECAYED || MODE == MODE_RETAIN) {
                    const uint64_t gg = pair_f32(head_decay, head_decay);
                    uint64_t vv[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) vv[c] = pair_f32(v[c], v[c]);
#pragma unroll
                    for (int m = 0; m < R / 2; ++m) {
                        const uint64_t f = MODE == MODE_DECAYED ? fr[MODE == MODE_DECAYED ? m : 0] : gg;
#pragma unroll
                        for (int c = 0; c < C; ++c) S[c][m] = fma_pair(kr[m], vv[c], mul_pair(f, S[c][m]));
                    }
                    if (tt > 0) reduce(tt - 1, false, nullptr);
                    if constexpr (MODE == MODE_DECAYED) fetch(fr, f4, next);
                } else {
                    const uint64_t ones = pair_f32(1.f, 1.f), neg = pair_f32(-1.f, -1.f);
                    uint64_t vv[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) vv[c] = pair_f32(v[c], v[c]);
#pragma unroll
                    for (int m = 0; m < R / 2; ++m) {
                        const uint64_t f = kr[m], nf = fma_pair(f, neg, ones);      // 1 - f
#pragma unroll
                        for (int c = 0; c < C; ++c) S[c][m] = fma_pair(f, S[c][m], mul_pair(nf, vv[c]));
                    }
                    if (tt > 0) reduce(tt - 1, false, nullptr);
                }
                fetch(kr, k4, next);
#pragma unroll
                for (int m = 0; m < R / 2; ++m) {
#pragma unroll
                    for (int c = 0; c < C; ++c) o2[c] = fma_pair(S[c][m], qr[m], o2[c]);
                }
                fetch(qr, q4, next);
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    float even, oddp;
                    unpair_f32(o2[c], even, oddp);
                    o_prev[c] = even + oddp;
                }
            }
            reduce(nb - 1, false, nullptr);
            group_barrier(2, WALKERS);
            float* orow = a.out + (size_t)(t0 + b0) * (a.H * dv) + h * dv + c0;
            for (int idx = tid; idx < nb * CT; idx += WALKERS) {
                const int tt = idx >> a.ct_shift, c = idx & (CT - 1);
                if (c0 + c < dv) orow[(size_t)tt * (a.H * dv) + c] = o_s[idx];
            }
        }
        if (stager && b + 1 < batches) {
            const int nn = min(TB, n - b0 - TB);
            if (one) stage_tokens<MODE, true, R>(a, stage_at((b + 1) & 1), ltid, h, hk, t0 + b0 + TB, nn, c0, pos0 + b0 + TB);
            else stage_tokens<MODE, false, R>(a, stage_at((b + 1) & 1), ltid, h, hk, t0 + b0 + TB, nn, c0, pos0 + b0 + TB);
        }
        __syncthreads();      // the walkers are done with this half and with o_s, the stagers have filled the other half
    }
    if (walker) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int j = c0 + cg * C + c;
#pragma unroll
            for (int m = 0; m < R / 4; ++m) {
                const int i = 4 * (kl + L * m);
                if (j < dv && i < d) {
                    float4 t;
                    unpair_f32(S[c][2 * m], t.x, t.y);
                    unpair_f32(S[c][2 * m + 1], t.z, t.w);
                    float* dst = st + (size_t)j * d + i;
                    if (vec) *reinterpret_cast<float4*>(dst) = t;
                    else {
                        dst[0] = t.x;
                        if (i + 1 < d) dst[1] = t.y;
                        if (i + 2 < d) dst[2] = t.z;
                        if (i + 3 < d) dst[3] = t.w;
                    }
                }
            }
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
        float v = o[base + c] * rstd * (w != nullptr ? w[c] : 1.f);
        if (gate.p != nullptr) v *= silu_f(rows_at(gate, t, gate_col + h * dv + c));
        out[base + c] = from_f32<TOUT>(v);
    }
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int MODE, int R, int C>
int rnn_launch(RnnArgs a, bool split, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = split ? matrix_rnn_kernel<MODE, true, R, C> : matrix_rnn_kernel<MODE, false, R, C>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        vcb_set_error("matrix_rnn: %zu bytes of shared memory refused", smem);
        return -2;
    }
    launch_pdl(kern, grid, dim3(split ? THREADS : WALKERS), smem, stream, a);
    return 0;
}

}  // namespace

// mode 0: the gated delta rule; 1: the gated linear form; 2: the decayed form; 3: retention (see the head of this file).
// u [S][T][ld] the projection's sums; x [T][ldx] the convolved rows (mode 0); z [zS][T][zld] the decay's sums (mode 2).
// state [slots][H][dv][d] (a value column's d rows in a run).  out [rows][H * dv] 32-bit, rows >= the entries' tokens.
// Entries of no tokens are left out.
VCB_API int vcb_matrix_rnn(int mode, const float* u, int S, long long s_stride, long long ld, const float* x, long long ldx,
                           int q_col, int k_col, int v_col, int b_col, int a_col, const float* dt_bias, const float* rate,
                           const float* f_bias, const float* lower, float* state, long long state_stride, const int* q_start,
                           const int* q_len, const int* slots, int E, int rows, int H, int G, int d, int dv, float* out,
                           const float* z, int zS, long long z_stride, long long zld, float inv_tau, const float* decay,
                           const int* ctx_len, const float* freq, int rot, int interleaved, cudaStream_t stream) {
    if (E == 0) return 0;
    VCB_CHECK_ARG(mode >= 0 && mode <= 3, "matrix_rnn: unknown mode %d", mode);
    VCB_CHECK_ARG(mode != 2 || (z != nullptr && f_bias != nullptr), "matrix_rnn: the decayed form needs the decay's sums and bias");
    VCB_CHECK_ARG(mode != 3 || (decay != nullptr && ctx_len != nullptr && rot >= 0 && rot <= d && rot % 2 == 0 && (rot == 0 || freq != nullptr)),
                  "matrix_rnn: retention needs a decay per head, the entries' positions and %d <= %d turning lanes with their frequencies", rot, d);
    VCB_CHECK_ARG(d >= 1 && d <= 512, "matrix_rnn: %d state rows a head (1 to 512)", d);
    VCB_CHECK_ARG(H >= 1 && G >= 1 && H % G == 0 && dv >= 1, "matrix_rnn: bad sizes H=%d G=%d dv=%d", H, G, dv);
    VCB_CHECK_ARG(H <= 65535 && E <= 65535, "matrix_rnn: %d heads, %d entries", H, E);
    VCB_CHECK_ARG(ld < (1 << 26) && ldx < (1 << 26), "matrix_rnn: rows of %lld and %lld lanes", ld, ldx);
    const int R = d <= 64 ? 8 : 16;     // rows a thread keeps of a column
    int L = 1;                          // lanes that share a column
    while (L * R < d) L <<= 1;
    // one column a thread while that gives no more blocks than there are SMs (a long portion of one request), else two
    const long long blocks1 = (long long)((dv + WALKERS / L - 1) / (WALKERS / L)) * H * E;
    const int C = blocks1 <= sm_count() ? 1 : 2;
    const int CT = C * WALKERS / L, DP = L * R;
    const int TB = DP <= 256 ? 16 : 8;
    int dp_shift = 0, ct_shift = 0;
    while ((1 << dp_shift) < DP) ++dp_shift;
    while ((1 << ct_shift) < CT) ++ct_shift;
    RnnArgs a{Rows{u, S < 1 ? 1 : S, s_stride, ld}, x, ldx, q_col, k_col, v_col, b_col, a_col, dt_bias, rate, f_bias, lower, state,
              state_stride, q_start, q_len, slots, out, H, G, d, dv, L, TB, dp_shift, ct_shift,
              Rows{z, zS < 1 ? 1 : zS, z_stride, zld}, inv_tau, decay, ctx_len, freq, rot, interleaved};
    const size_t smem = (size_t)(2 * ((mode == 2 ? 3 : 2) * TB * DP + TB * CT + 2 * TB) + TB * CT) * sizeof(float);
    const dim3 grid((dv + CT - 1) / CT, H, E);
    const bool split = rows > 4 * E;    // some entry has more than four tokens
    int rc;
#define VCB_RNN_GO(MODE_, R_) (C == 1 ? rnn_launch<MODE_, R_, 1>(a, split, grid, smem, stream) : rnn_launch<MODE_, R_, 2>(a, split, grid, smem, stream))
    if (R == 8) rc = mode == 0 ? VCB_RNN_GO(MODE_DELTA, 8) : mode == 1 ? VCB_RNN_GO(MODE_GATED, 8) : mode == 2 ? VCB_RNN_GO(MODE_DECAYED, 8) : VCB_RNN_GO(MODE_RETAIN, 8);
    else rc = mode == 0 ? VCB_RNN_GO(MODE_DELTA, 16) : mode == 1 ? VCB_RNN_GO(MODE_GATED, 16) : mode == 2 ? VCB_RNN_GO(MODE_DECAYED, 16) : VCB_RNN_GO(MODE_RETAIN, 16);
#undef VCB_RNN_GO
    if (rc != 0) return rc;
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
