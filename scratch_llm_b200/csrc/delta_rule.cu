// The gated delta rule: a linear recurrence whose state is one matrix S [D, V] per head and
// request, carried in 32-bit from token to token.  Per token, with a unit key k and a scaled
// unit query q of size D, a value v of size V, a decay g in (0, 1) and a step size beta:
//
//     S  <-  g S
//     u   =  beta (v - S^T k)
//     S  <-  S + k u^T
//     o   =  S^T q                       (the read-out sees the token's own write)
//
// with, computed here in 32-bit from what the projections and the short convolution left:
//     k = k_raw / sqrt(sum(k_raw^2) + 1e-6),   q = q_raw / sqrt(sum(q_raw^2) + 1e-6) * D^(-1/2)
//     beta = sigmoid(b),   g = exp(-exp(A_log) * softplus(a + dt_bias))
// Head h of H reads key/query head h / (H / G).
//
// Columns of S are independent of each other: u_j and o_j need column j of S only.  A warp
// owns one column (its 32 lanes hold D / 32 elements each, in quads), a CTA of 16 warps takes
// 16 columns of one (row, head).  Tokens are taken in chunks of TC = 16, and inside a chunk the
// recurrence is unrolled so that only a small triangular system is sequential.  With S0 the
// state at the chunk's start, L_t the sum of log g up to token t of the chunk, per column:
//
//     p_t = S0^T k_t,  r_t = S0^T q_t                          (independent dot products)
//     u_t = beta_t ( v_t - e^{L_t} p_t - sum_{s<t} e^{L_t - L_s} (k_s . k_t) u_s )
//     o_t = e^{L_t} r_t + sum_{s<=t} e^{L_t - L_s} (k_s . q_t) u_s
//     S   = e^{L_last} S0 + sum_s e^{L_last - L_s} k_s u_s^T
//
// which is the rule above written out (S'_t = e^{L_t} S0 + sum_{s<t} e^{L_t - L_s} k_s u_s^T).
// The CTA norms the chunk's keys and queries, evaluates its gates and the table of weighted dot
// products once (all of this is shared by its 16 columns).  A warp then forms its 32 partial
// dot products with S0, sums them across its lanes so that lane t holds p_t and lane 16 + t
// holds r_t (31 shuffles), and solves the triangular system column by column: lane s
// announces u_s, every lane adds its row's weight times u_s to its own sum, so that the lanes
// 16 + t end with the read-outs o_t.  Last comes the rank-16 update of its elements of S.
// All of it is 32-bit.  A chunk's inputs are requested one chunk ahead and wait in registers.
// The same kernel serves portions of prompts (many tokens per row) and decoding (a chunk of one
// token); a row reads its state from its slot and writes it back; rows without tokens touch
// nothing.
//
//
// A decay per key CHANNEL (log_decay != null: float [tokens, H * D], the logarithm of each
// channel's factor, at most 0): S <- diag(g) S in the rule's first line.  With L_t now the vector
// of the channels' sums of log g up to token t of the chunk, the same unrolling holds with
//     p_t = S0^T (e^{L_t} * k_t),   r_t = S0^T (e^{L_t} * q_t),
//     weights  sum_d k_s[d] x_t[d] e^{L_t[d] - L_s[d]}   (x = k for s < t, x = q for s <= t),
//     S = diag(e^{L_last}) S0 + sum_s (e^{L_last - L_s} * k_s) u_s^T.
// Every exponent that is formed is at most 0 (a later token's sum minus an earlier one's), so
// nothing overflows however strong the decay; the weights cost one exponential per channel and
// pair of tokens, shared by the CTA's 16 columns.  The step size then comes from column b_col +
// head of `ab`, and A_log / dt_bias are the caller's business (they are inside log_decay).
//
// The weights depend on keys, queries and decays alone: delta_weights_kernel forms the tables of
// ALL chunks of a step in parallel before the scan starts, which then reads its chunk's table.
//
// Compiled once per key size: -DSLLM_HEAD_DIM=<D>.
#include "common.cuh"

#ifndef SLLM_HEAD_DIM
#error "compile with -DSLLM_HEAD_DIM=<key size>"
#endif

namespace sllm {

constexpr int D = SLLM_HEAD_DIM;
static_assert(D >= 1 && D <= 256, "key size: 1 to 256 (a chunk of keys and queries is staged in shared memory)");
constexpr int QUADS = (D + 3) / 4;                  // groups of 4 elements of a column
constexpr int QPL = (QUADS + 31) / 32;              // quads per lane
constexpr int LDK = 4 * QUADS + 4;                  // row stride of the staged keys / queries
constexpr int TC = 16;                              // tokens per chunk
constexpr int COLS = 16;                            // columns (warps) per CTA
constexpr int THREADS = 32 * COLS;

struct DeltaArgs {
    const void* act; int64_t ld_act;     // [tokens, >= 2 G D + H V]: q heads, k heads, v heads
    const float* ab; int64_t ld_ab;      // [tokens, >= 2 H]: a (decay input) then b (step input)
    const float* A_log; const float* dt_bias;   // [H]
    float* state;                        // [slots, H, V, D]
    const int* row_start; const int* row_slot;
    float* out;                          // [tokens, H * V]
    int H; int G; int V;
    // a decay per key channel: [tokens, >= H * D] logarithms (null: one decay per head from a)
    const float* log_decay; int64_t ld_decay;
    int b_col;                           // the step input of head h is ab[b_col + h]
    // with a decay per channel: the chunks' tables of weights, made by delta_weights_kernel before
    // this launch (null: every CTA forms its chunk's table itself).  The chunk that starts at
    // token t of row r has slot t / TC + r; a slot holds [H][2 TC][TC] floats.
    const float* tables;
};
// the kernel for a decay per channel stages a third [TC][D] table in (static) shared memory
constexpr bool CHANNEL_FITS = D <= 192;

// One token of one column by one warp: the rule as it stands.  Every warp norms the key and
// the query itself (its lanes hold the same quads of them as of its column).  S: the lane's
// elements of the column (already loaded), st: where they live.
template <typename T, bool CHANNEL>
__device__ __forceinline__ void single_token(const DeltaArgs& a, float* S, float* st, int t0,
                                             int head, int g, int col, bool live, int lane) {
    const T* act = reinterpret_cast<const T*>(a.act);
    const int64_t k_col0 = (int64_t)a.G * D, v_col0 = 2 * (int64_t)a.G * D;
    const float decay_rate = CHANNEL ? 0.f : expf(a.A_log[head]);
    const float dt_bias = CHANNEL ? 0.f : a.dt_bias[head];
    const float q_scale = rsqrtf((float)D);
        float kq[4 * QPL], qq[4 * QPL];
        float sk = 0.f, sq = 0.f;
        const T* row = act + (int64_t)t0 * a.ld_act + (int64_t)g * D;
#pragma unroll
        for (int i = 0; i < QPL; ++i)
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int e = (i * 32 + lane) * 4 + w;
                kq[4 * i + w] = e < D ? to_float(row[k_col0 + e]) : 0.f;
                qq[4 * i + w] = e < D ? to_float(row[e]) : 0.f;
                sk += kq[4 * i + w] * kq[4 * i + w];
                sq += qq[4 * i + w] * qq[4 * i + w];
            }
        sk = warp_sum(sk);
        sq = warp_sum(sq);
        const float ik = 1.0f / sqrtf(sk + 1e-6f), iq = q_scale / sqrtf(sq + 1e-6f);
        const float* ab = a.ab + (int64_t)t0 * a.ld_ab;
        float decay = 1.f;
        if (CHANNEL) {      // this lane's channels fade by their own factors
            const float* lg = a.log_decay + (int64_t)t0 * a.ld_decay + (int64_t)head * D;
#pragma unroll
            for (int i = 0; i < QPL; ++i)
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int e = (i * 32 + lane) * 4 + w;
                    if (e < D) S[4 * i + w] *= expf(lg[e]);
                }
        } else {
            const float x = ab[head] + dt_bias;
            decay = expf(-decay_rate * (x > 20.f ? x : log1pf(expf(x))));
        }
        const float beta = 1.0f / (1.0f + expf(-ab[a.b_col + head]));
        const float value = live ? to_float(act[(int64_t)t0 * a.ld_act + v_col0 +
                                                (int64_t)head * a.V + col]) : 0.f;
        float p = 0.f, rq = 0.f, kdq = 0.f;
#pragma unroll
        for (int i = 0; i < 4 * QPL; ++i) {
            kq[i] *= ik;
            qq[i] *= iq;
            if (!CHANNEL) S[i] *= decay;
            p = fmaf(S[i], kq[i], p);
            rq = fmaf(S[i], qq[i], rq);
            kdq = fmaf(kq[i], qq[i], kdq);
        }
        p = warp_sum(p);
        rq = warp_sum(rq);
        kdq = warp_sum(kdq);
        const float u1 = beta * (value - p);
        if (live) {
            if (lane == 0)
                a.out[(int64_t)t0 * a.H * a.V + (int64_t)head * a.V + col] = rq + u1 * kdq;
#pragma unroll
            for (int i = 0; i < QPL; ++i)
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int e = (i * 32 + lane) * 4 + w;
                    if (e < D) st[e] = fmaf(kq[4 * i + w], u1, S[4 * i + w]);
                }
        }
}

// Steps in which every row brings one token (decoding): 4 warps = 4 columns per CTA, few
// registers, so that many CTAs share an SM and the states stream at the memory's rate.
constexpr int STEP_COLS = 4;
template <typename T, bool CHANNEL>
__global__ void __launch_bounds__(32 * STEP_COLS) delta_rule_step_kernel(const DeltaArgs a) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.z, head = blockIdx.y;
    const int t0 = a.row_start[r], n_new = a.row_start[r + 1] - t0;
    if (n_new <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * STEP_COLS + warp;
    const bool live = col < a.V;
    float S[4 * QPL];
    float* st = a.state + (((int64_t)a.row_slot[r] * a.H + head) * a.V + (live ? col : 0)) * D;
#pragma unroll
    for (int i = 0; i < QPL; ++i) {
        const int e = (i * 32 + lane) * 4;
        if (live && D % 4 == 0 && e < D) {
            const float4 v = *reinterpret_cast<const float4*>(st + e);
            S[4 * i] = v.x; S[4 * i + 1] = v.y; S[4 * i + 2] = v.z; S[4 * i + 3] = v.w;
        } else {
#pragma unroll
            for (int w = 0; w < 4; ++w) S[4 * i + w] = (live && e + w < D) ? st[e + w] : 0.f;
        }
    }
    single_token<T, CHANNEL>(a, S, st, t0, head, head / (a.H / a.G), col, live, lane);
}

// VECTOR: keys and queries are fetched in 16-byte pieces (D a multiple of 16 / sizeof(T), rows
// and base 16-byte aligned); else element by element.
template <typename T, bool VECTOR, bool CHANNEL>
__global__ void __launch_bounds__(THREADS) delta_rule_kernel(const DeltaArgs a) {
    constexpr int VEC = VECTOR ? 16 / (int)sizeof(T) : 1;
    constexpr int PER_ROW = D / VEC;                               // pieces of a key or query
    constexpr int QK_PIECES = 2 * TC * PER_ROW;                    // of a chunk
    constexpr int QK_ITEMS = (QK_PIECES + THREADS - 1) / THREADS;  // per thread
    struct alignas(16) Piece { T e[VEC]; };
    // keys and queries of the chunk as unit vectors (the query scaled), padded with zeros to
    // whole quads; lane l of a warp owns the quads l, l + 32, ... of its column
    __shared__ __align__(16) float ks[TC][LDK];
    __shared__ __align__(16) float qs[TC][LDK];
    __shared__ float vs[TC][COLS];
    // row t < 16: -e^{L_t - L_s} (k_s . k_t) for s < t; row 16 + t: e^{L_t - L_s} (k_s . q_t) for
    // s <= t; zero elsewhere
    __shared__ float weight[2 * TC][TC + 1];
    __shared__ float log_g[TC], cum_s[TC], beta_s[TC], grow_s[TC], rest_s[TC];
    // a decay per channel: the channels' log decays of the chunk's tokens, then their running
    // sums L_t, and at last e^{L_t} * k_t (the keys that meet S0); last_s: L of the chunk's last token
    __shared__ __align__(16) float lam[CHANNEL ? TC : 1][CHANNEL ? LDK : 4];
    __shared__ float last_s[CHANNEL ? LDK : 4];

    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.z, head = blockIdx.y;
    const int t0 = a.row_start[r], n_new = a.row_start[r + 1] - t0;
    if (n_new <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = head / (a.H / a.G);
    const int col0 = blockIdx.x * COLS;
    const int col = col0 + warp;
    const bool live = col < a.V;
    const T* act = reinterpret_cast<const T*>(a.act);
    const int64_t k_col0 = (int64_t)a.G * D, v_col0 = 2 * (int64_t)a.G * D;

    float S[4 * QPL];
    float* st = a.state + (((int64_t)a.row_slot[r] * a.H + head) * a.V + (live ? col : 0)) * D;
#pragma unroll
    for (int i = 0; i < QPL; ++i)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int e = (i * 32 + lane) * 4 + w;
            S[4 * i + w] = (live && e < D) ? st[e] : 0.f;
        }
    const float decay_rate = CHANNEL ? 0.f : expf(a.A_log[head]);
    const float dt_bias = CHANNEL ? 0.f : a.dt_bias[head];
    const float q_scale = rsqrtf((float)D);

    if (n_new == 1) {   // decoding: no shared memory, no barrier
        single_token<T, CHANNEL>(a, S, st, t0, head, g, col, live, lane);
        return;
    }
    // columns beyond D (where D is no multiple of 4) stay zero for good
    for (int idx = tid; idx < TC * LDK; idx += THREADS) {
        (&ks[0][0])[idx] = 0.f;
        (&qs[0][0])[idx] = 0.f;
        if (CHANNEL) (&lam[0][0])[idx] = 0.f;
    }
    if (CHANNEL && tid < LDK) last_s[tid] = 0.f;
    Piece raw[QK_ITEMS];
    T raw_v = from_float<T>(0.f);
    float raw_a = 0.f, raw_b = 0.f;
    // a decay per channel: the chunk's log decays and this thread's entry of its table of weights
    // travel with the same request
    constexpr int L_ITEMS = CHANNEL ? (TC * D + THREADS - 1) / THREADS : 1;
    float raw_l[L_ITEMS], raw_w = 0.f;
    auto fetch = [&](int c0) {     // requests the chunk at c0 (tokens beyond the row: nothing)
        const int nt = min(TC, n_new - c0);
        if (CHANNEL) {
            const float* lg = a.log_decay + (int64_t)(t0 + c0) * a.ld_decay + (int64_t)head * D;
#pragma unroll
            for (int i = 0; i < L_ITEMS; ++i) {
                const int idx = tid + i * THREADS, t = idx / D, e = idx - t * D;
                raw_l[i] = (idx < TC * D && t < nt) ? lg[(int64_t)t * a.ld_decay + e] : 0.f;
            }
            if (a.tables != nullptr)
                raw_w = a.tables[(((int64_t)(t0 + c0) / TC + r) * a.H + head) * 2 * TC * TC + tid];
        }
#pragma unroll
        for (int i = 0; i < QK_ITEMS; ++i) {
            const int item = tid + i * THREADS;
            const int which = item / (TC * PER_ROW), rem = item - which * (TC * PER_ROW);
            const int t = rem / PER_ROW, c = rem - t * PER_ROW;
            if (item < QK_PIECES && t < nt) {
                const T* src = act + (int64_t)(t0 + c0 + t) * a.ld_act + (int64_t)g * D +
                               (which ? k_col0 : 0) + c * VEC;
                if (VECTOR) raw[i] = *reinterpret_cast<const Piece*>(src);
                else raw[i].e[0] = src[0];
            }
        }
        if (tid < TC * COLS) {
            const int t = tid / COLS, j = tid - t * COLS;
            if (t < nt && col0 + j < a.V)
                raw_v = act[(int64_t)(t0 + c0 + t) * a.ld_act + v_col0 + (int64_t)head * a.V +
                            col0 + j];
        }
        if (tid < nt) {
            const float* ab = a.ab + (int64_t)(t0 + c0 + tid) * a.ld_ab;
            raw_a = CHANNEL ? 0.f : ab[head];
            raw_b = ab[a.b_col + head];
        }
    };
    auto commit = [&](int nt) {    // what fetch() requested, into shared memory as 32-bit
#pragma unroll
        for (int i = 0; i < QK_ITEMS; ++i) {
            const int item = tid + i * THREADS;
            const int which = item / (TC * PER_ROW), rem = item - which * (TC * PER_ROW);
            const int t = rem / PER_ROW, c = rem - t * PER_ROW;
            if (item < QK_PIECES) {
                float* dst = (which ? &ks[t][0] : &qs[t][0]) + c * VEC;
#pragma unroll
                for (int w = 0; w < VEC; ++w) dst[w] = t < nt ? to_float(raw[i].e[w]) : 0.f;
            }
        }
        if (tid < TC * COLS) {
            const int t = tid / COLS, j = tid - t * COLS;
            vs[t][j] = (t < nt && col0 + j < a.V) ? to_float(raw_v) : 0.f;
        }
        if (tid < TC) {
            float lg = 0.f, beta = 0.f;
            if (tid < nt) {
                const float x = raw_a + dt_bias;
                const float softplus = x > 20.f ? x : log1pf(expf(x));
                lg = -decay_rate * softplus;                 // log of the decay
                beta = 1.0f / (1.0f + expf(-raw_b));
            }
            log_g[tid] = lg;
            beta_s[tid] = beta;
        }
    };
    __syncthreads();
    fetch(0);

    for (int c0 = 0; c0 < n_new; c0 += TC) {
        const int nt = min(TC, n_new - c0);
        __syncthreads();   // the previous chunk's staging is no longer read
        commit(nt);
        float table_entry = 0.f;
        if (CHANNEL) {     // the chunk's log decays per channel (zeros beyond its tokens)
#pragma unroll
            for (int i = 0; i < L_ITEMS; ++i) {
                const int idx = tid + i * THREADS, t = idx / D, e = idx - t * D;
                if (idx < TC * D) lam[t][e] = raw_l[i];
            }
            table_entry = raw_w;
        }
        if (c0 + TC < n_new) fetch(c0 + TC);   // in flight while this chunk is worked on
        __syncthreads();
        // unit vectors and the query's scale: one warp per token
        if (warp < nt) {
            const int t = warp;
            float sk = 0.f, sq = 0.f;
            for (int e = lane; e < D; e += 32) {
                sk += ks[t][e] * ks[t][e];
                sq += qs[t][e] * qs[t][e];
            }
            sk = warp_sum(sk);
            sq = warp_sum(sq);
            const float ik = 1.0f / sqrtf(sk + 1e-6f), iq = q_scale / sqrtf(sq + 1e-6f);
            for (int e = lane; e < D; e += 32) {
                ks[t][e] *= ik;
                qs[t][e] *= iq;
            }
        }
        if (CHANNEL) {               // running sums of the log decays, channel by channel
            // (warps nt .. 15 have no token to norm; with a full chunk everyone shares the work)
            for (int e = tid; e < D; e += THREADS) {
                float c = 0.f;
#pragma unroll
                for (int t = 0; t < TC; ++t) {
                    c += lam[t][e];
                    lam[t][e] = c;
                }
                last_s[e] = lam[nt - 1][e];
            }
        } else if (tid >= THREADS - TC) {   // (the last warp: it has no token to norm unless nt is 16)
            const int t = tid - (THREADS - TC);
            float c = 0.f, last = 0.f;
            for (int i = 0; i < TC; ++i) {
                if (i <= t) c += log_g[i];
                if (i < nt) last += log_g[i];
            }
            cum_s[t] = c;
            grow_s[t] = expf(c);            // e^{L_t}
            rest_s[t] = expf(last - c);     // e^{L_last - L_t}
        }
        __syncthreads();
        // the table of weights: thread -> (row, s); rows 0..15 pair keys with keys, 16..31 keys
        // with queries
        {
            const int row = tid >> 4, s = tid & 15, t = row & 15;
            const bool with_q = row >= TC;
            float dot = 0.f;
            const bool used = t < nt && s < nt && (with_q ? s <= t : s < t);
            if (CHANNEL && a.tables != nullptr) {
                dot = table_entry;       // (entry [row][s] = [tid / TC][tid % TC], as requested)
            } else if (used && CHANNEL) {
                const float* x = with_q ? &qs[t][0] : &ks[t][0];
                for (int e = 0; e < D; ++e)
                    dot = fmaf(x[e] * ks[s][e], expf(lam[t][e] - lam[s][e]), dot);
            } else if (used) {
                const float* x = with_q ? &qs[t][0] : &ks[t][0];
#pragma unroll 4
                for (int c = 0; c < QUADS; ++c) {
                    const float4 xa = *reinterpret_cast<const float4*>(x + 4 * c);
                    const float4 kb = *reinterpret_cast<const float4*>(&ks[s][4 * c]);
                    dot += xa.x * kb.x + xa.y * kb.y + xa.z * kb.z + xa.w * kb.w;
                }
                dot *= expf(cum_s[t] - cum_s[s]);
            }
            weight[row][s] = with_q ? dot : -dot;
        }
        __syncthreads();
        if (CHANNEL) {
            // what the rest of the chunk needs: e^{L_t} * k_t (in lam's place) and e^{L_t} * q_t for
            // the products with S0, and e^{L_last - L_t} * k_t for the state's update
            for (int idx = tid; idx < TC * D; idx += THREADS) {
                const int t = idx / D, e = idx - t * D;
                const float L = lam[t][e], grow = expf(L), k = ks[t][e];
                lam[t][e] = grow * k;
                qs[t][e] *= grow;
                ks[t][e] = t < nt ? k * expf(last_s[e] - L) : 0.f;
            }
            __syncthreads();
        }

        // ---- this lane's share of S0^T k_t (v[t]) and S0^T q_t (v[16 + t])
        float v[2 * TC];
#pragma unroll
        for (int t = 0; t < TC; ++t) {
            float pk = 0.f, pq = 0.f;
#pragma unroll
            for (int i = 0; i < QPL; ++i) {
                const int c = i * 32 + lane;
                if (c < QUADS) {
                    const float4 kt = *reinterpret_cast<const float4*>(
                        CHANNEL ? &lam[t][4 * c] : &ks[t][4 * c]);
                    const float4 qt = *reinterpret_cast<const float4*>(&qs[t][4 * c]);
                    pk += S[4 * i] * kt.x + S[4 * i + 1] * kt.y + S[4 * i + 2] * kt.z +
                          S[4 * i + 3] * kt.w;
                    pq += S[4 * i] * qt.x + S[4 * i + 1] * qt.y + S[4 * i + 2] * qt.z +
                          S[4 * i + 3] * qt.w;
                }
            }
            v[t] = pk;
            v[TC + t] = pq;
        }
        // ---- sum over the lanes, so that lane i ends with the total of v[i]: in the round
        // with offset o a lane keeps the half of its values whose index has bit o as its own
        // lane number has, and hands the other half to its partner
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const bool upper = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < o; ++i) {
                const float give = upper ? v[i] : v[i + o];
                const float keep = upper ? v[i + o] : v[i];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, give, o);
            }
        }
        // lane t < 16: the sum that becomes u_t; lane 16 + t: the sum that becomes o_t
        const int t_mine = lane & 15;
        const float grow_mine = CHANNEL ? 1.f : grow_s[t_mine];   // (per channel: inside v[0])
        float acc = lane < TC ? vs[t_mine][warp] - grow_mine * v[0] : grow_mine * v[0];
        const float beta_mine = lane < TC ? beta_s[t_mine] : 0.f;
        float u[TC];
#pragma unroll
        for (int s = 0; s < TC; ++s) {
            u[s] = __shfl_sync(0xffffffffu, beta_mine * acc, s);   // lane s has all of its sum
            acc = fmaf(weight[lane][s], u[s], acc);                 // (weight[s][s] is 0)
        }
        if (lane >= TC && t_mine < nt && live)
            a.out[(int64_t)(t0 + c0 + t_mine) * a.H * a.V + (int64_t)head * a.V + col] = acc;
        // ---- the state after the chunk
        if (CHANNEL) {
#pragma unroll
            for (int i = 0; i < QPL; ++i)
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int e = (i * 32 + lane) * 4 + w;
                    if (e < D) S[4 * i + w] *= expf(last_s[e]);
                }
        } else {
            const float keep_all = grow_s[nt - 1];
#pragma unroll
            for (int i = 0; i < 4 * QPL; ++i) S[i] *= keep_all;
        }
#pragma unroll
        for (int t = 0; t < TC; ++t) {
            // (u is zero beyond the chunk's tokens; per channel the keys carry their factors)
            const float f = CHANNEL ? u[t] : rest_s[t] * u[t];
#pragma unroll
            for (int i = 0; i < QPL; ++i) {
                const int c = i * 32 + lane;
                if (c < QUADS) {
                    const float4 kt = *reinterpret_cast<const float4*>(&ks[t][4 * c]);
                    S[4 * i] = fmaf(kt.x, f, S[4 * i]);
                    S[4 * i + 1] = fmaf(kt.y, f, S[4 * i + 1]);
                    S[4 * i + 2] = fmaf(kt.z, f, S[4 * i + 2]);
                    S[4 * i + 3] = fmaf(kt.w, f, S[4 * i + 3]);
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < QPL; ++i)
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int e = (i * 32 + lane) * 4 + w;
                if (e < D) st[e] = S[4 * i + w];
            }
    }
}

// The tables of weights of all chunks of a step at once, for a decay per channel (the comment at
// the top): they depend on the keys, queries and decays alone, not on the state, so the chunks of
// a row need not wait for each other.  grid (chunks of the longest row, H, rows), 256 threads: a
// thread per pair of tokens that the table uses (120 pairs of keys with earlier keys, 136 of
// queries with keys up to their own).  tables: [slots][H][2 TC][TC] as DeltaArgs says; entries
// that no pair uses are zero.
constexpr int TABLE_THREADS = 256;
template <typename T>
__global__ void __launch_bounds__(TABLE_THREADS) delta_weights_kernel(const DeltaArgs a, float* tables) {
    __shared__ __align__(16) float ks[TC][LDK];
    __shared__ __align__(16) float qs[TC][LDK];
    __shared__ __align__(16) float lam[TC][LDK];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.z, head = blockIdx.y, c0 = blockIdx.x * TC;
    const int t0 = a.row_start[r], n_new = a.row_start[r + 1] - t0;
    if (c0 >= n_new || n_new <= 1) return;     // (rows of one token take the kernel's plain path)
    const int nt = min(TC, n_new - c0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = head / (a.H / a.G);
    const T* act = reinterpret_cast<const T*>(a.act);
    const int64_t k_col0 = (int64_t)a.G * D;
    for (int idx = tid; idx < TC * D; idx += TABLE_THREADS) {
        const int t = idx / D, e = idx - t * D;
        float k = 0.f, q = 0.f, l = 0.f;
        if (t < nt) {
            const T* row = act + (int64_t)(t0 + c0 + t) * a.ld_act + (int64_t)g * D;
            q = to_float(row[e]);
            k = to_float(row[k_col0 + e]);
            l = a.log_decay[(int64_t)(t0 + c0 + t) * a.ld_decay + (int64_t)head * D + e];
        }
        ks[t][e] = k; qs[t][e] = q; lam[t][e] = l;
    }
    __syncthreads();
    const float q_scale = rsqrtf((float)D);
    for (int t = warp; t < nt; t += TABLE_THREADS / 32) {
        float sk = 0.f, sq = 0.f;
        for (int e = lane; e < D; e += 32) {
            sk += ks[t][e] * ks[t][e];
            sq += qs[t][e] * qs[t][e];
        }
        sk = warp_sum(sk);
        sq = warp_sum(sq);
        const float ik = 1.0f / sqrtf(sk + 1e-6f), iq = q_scale / sqrtf(sq + 1e-6f);
        for (int e = lane; e < D; e += 32) {
            ks[t][e] *= ik;
            qs[t][e] *= iq;
        }
    }
    for (int e = tid; e < D; e += TABLE_THREADS) {
        float c = 0.f;
#pragma unroll
        for (int t = 0; t < TC; ++t) {
            c += lam[t][e];
            lam[t][e] = c;
        }
    }
    __syncthreads();
    float* table = tables + (((int64_t)(t0 + c0) / TC + r) * a.H + head) * 2 * TC * TC;
    // thread -> pair: the first 120 threads take (t, s < t) of keys with keys, the other 136 take
    // (t, s <= t) of queries with keys; both triangles are walked row by row
    const bool with_q = tid >= TC * (TC - 1) / 2;
    int p = with_q ? tid - TC * (TC - 1) / 2 : tid, t = 0;
    if (with_q) { while (p > t) { p -= t + 1; ++t; } }        // row t has t + 1 pairs
    else { t = 1; while (p >= t) { p -= t; ++t; } }           // row t has t pairs
    const int sidx = p;
    float dot = 0.f;
    if (t < nt) {
        const float* x = with_q ? &qs[t][0] : &ks[t][0];
#pragma unroll 4
        for (int e = 0; e < D; ++e)
            dot = fmaf(x[e] * ks[sidx][e], __expf(lam[t][e] - lam[sidx][e]), dot);
    }
    table[((with_q ? TC : 0) + t) * TC + sidx] = dot;
    // the entries that no pair uses
    for (int idx = tid; idx < 2 * TC * TC; idx += TABLE_THREADS) {
        const int row = idx / TC, s2 = idx - row * TC, t2 = row & (TC - 1);
        if (row >= TC ? s2 > t2 : s2 >= t2) table[idx] = 0.f;
    }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_delta_rule_head_dim() { return D; }

// dtype: 0 = float32, 1 = bfloat16 (of act).  n_rows rows of the packed batch (row_start has
// n_rows + 1 entries); state slots are indexed by row_slot.  max_new: the most tokens any row
// brings (1 selects the kernel for decode steps).
SLLM_EXPORT int sllm_delta_rule(const void* act, int64_t ld_act, const float* ab, int64_t ld_ab,
                                const float* A_log, const float* dt_bias, float* state,
                                const int* row_start, const int* row_slot, float* out, int n_rows,
                                int max_new, int H, int G, int V, const float* log_decay,
                                int64_t ld_decay, int b_col, float* tables, int longest,
                                int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || V <= 0 || n_rows > 65535 || H > 65535 ||
        ld_act < 2 * (int64_t)G * D + (int64_t)H * V || b_col < 0 || ld_ab < b_col + H ||
        (!log_decay && (ld_ab < H || !A_log || !dt_bias)) ||
        (log_decay && (ld_decay < (int64_t)H * D || !CHANNEL_FITS)))
        return (int)cudaErrorInvalidValue;
    DeltaArgs a;
    a.log_decay = log_decay; a.ld_decay = ld_decay; a.b_col = b_col;
    a.tables = nullptr;
    a.act = act; a.ld_act = ld_act; a.ab = ab; a.ld_ab = ld_ab; a.A_log = A_log;
    a.dt_bias = dt_bias; a.state = state; a.row_start = row_start; a.row_slot = row_slot;
    a.out = out; a.H = H; a.G = G; a.V = V;
    if (max_new == 1) {   // no row brings more than one token
        dim3 sgrid((V + STEP_COLS - 1) / STEP_COLS, H, n_rows);
        if (dtype != 0 && dtype != 1) return (int)cudaErrorInvalidValue;
        if (log_decay) {
            if (dtype == 0) delta_rule_step_kernel<float, true><<<sgrid, 32 * STEP_COLS, 0, stream>>>(a);
            else delta_rule_step_kernel<__nv_bfloat16, true><<<sgrid, 32 * STEP_COLS, 0, stream>>>(a);
        } else {
            if (dtype == 0) delta_rule_step_kernel<float, false><<<sgrid, 32 * STEP_COLS, 0, stream>>>(a);
            else delta_rule_step_kernel<__nv_bfloat16, false><<<sgrid, 32 * STEP_COLS, 0, stream>>>(a);
        }
        SLLM_LAUNCH_CHECK();
        return 0;
    }
    dim3 grid((V + COLS - 1) / COLS, H, n_rows);
    const size_t esize = dtype == 0 ? 4 : 2;
    const int vec = (int)(16 / esize);
    // 16-byte pieces need every key, query and row of `act` to start on a 16-byte boundary
    const bool vector = D % vec == 0 && ld_act % vec == 0 && ((uintptr_t)act & 15) == 0 &&
                        ((int64_t)G * D) % vec == 0;
    if (dtype != 0 && dtype != 1) return (int)cudaErrorInvalidValue;
    if (log_decay) {
        if constexpr (CHANNEL_FITS) {
            if (tables != nullptr && longest > 1) {
                // all chunks' tables at once; `tables` holds (tokens / TC + n_rows + 1) slots of
                // H * 2 TC * TC floats, `longest` is the most tokens any row brings
                dim3 tgrid((longest + TC - 1) / TC, H, n_rows);
                if (tgrid.x > 65535u * 32u) return (int)cudaErrorInvalidValue;
                if (dtype == 0) delta_weights_kernel<float><<<tgrid, TABLE_THREADS, 0, stream>>>(a, tables);
                else delta_weights_kernel<__nv_bfloat16><<<tgrid, TABLE_THREADS, 0, stream>>>(a, tables);
                SLLM_LAUNCH_CHECK();
                a.tables = tables;
            }
            if (dtype == 0) {
                if (vector) delta_rule_kernel<float, (D % 4 == 0), true><<<grid, THREADS, 0, stream>>>(a);
                else delta_rule_kernel<float, false, true><<<grid, THREADS, 0, stream>>>(a);
            } else {
                if (vector) delta_rule_kernel<__nv_bfloat16, (D % 8 == 0), true><<<grid, THREADS, 0, stream>>>(a);
                else delta_rule_kernel<__nv_bfloat16, false, true><<<grid, THREADS, 0, stream>>>(a);
            }
        }
    } else if (dtype == 0) {
        if (vector) delta_rule_kernel<float, (D % 4 == 0), false><<<grid, THREADS, 0, stream>>>(a);
        else delta_rule_kernel<float, false, false><<<grid, THREADS, 0, stream>>>(a);
    } else {
        if (vector) delta_rule_kernel<__nv_bfloat16, (D % 8 == 0), false><<<grid, THREADS, 0, stream>>>(a);
        else delta_rule_kernel<__nv_bfloat16, false, false><<<grid, THREADS, 0, stream>>>(a);
    }
    SLLM_LAUNCH_CHECK();
    return 0;
}
