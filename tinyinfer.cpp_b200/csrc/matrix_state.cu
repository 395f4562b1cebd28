// Recurrent mixers whose per-head state is a matrix S [dk keys, dv values] in float32, kept per
// request in a state slot and carried from token to token.
//
//  * MODE_DELTA, the gated delta rule.  Per token, with k and q brought to unit length over the head
//    (x / sqrt(sum x^2 + 1e-6); q also times dk^-1/2), beta = sigmoid(b), and the decay
//    g = exp(-exp(A_log_h) * softplus(a + dt_bias_h)):
//        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
//  * MODE_GATED_SUM, a matrix memory with exponential gates kept finite by a running maximum m
//    (m = 0 at the start).  With log gates i = cap tanh((zi + bi) / cap) and
//    f = logsigmoid(cap tanh((zf + bf) / cap)):
//        m' = max(f + m, i);   S <- e^(f + m - m') S + e^(i - m') k v^T;   n likewise with k alone;
//        o = S^T q / (max(|n . q|, e^(-m')) + 1e-6),   q times dk^-1/2.
//    n rides as one more column of S whose value is always 1.
//
// Both then bring each head's o to unit root mean square over dv, multiply by a weight (one per
// element of a head, or one per element of the row) and by act(gate) (silu or sigmoid), and write
// the row in the activation dtype.
//
// One block walks the tokens of one (request, head) in order.  A column of S is spread over the rows:
// sixteen "virtual lanes" each own four rows of every 64 (rows 64 g + 4 lane + 0..3), and a sum over
// the rows is always taken per virtual lane first and then over the lanes as a tree of pairs
// (lane ^ 1, ^ 2, ^ 4, ^ 8).  A thread plays four virtual lanes when a head's columns sit in one
// block (4 threads a column, up to 128 columns), or one when the columns are cut over several blocks
// (16 threads a column, 8 to 32 columns a block: few requests with long portions, where the walk is
// bound by the instructions a warp issues per token); the bits are the same either way.  Blocks of
// cut columns write o as float32 and leave the norm, the weight and the gate to
// `matrix_state_finish`.  In the gated sum every such block reads the normaliser's column and the
// running maximum, so their new values wait in `carry` until all blocks are through and a small
// launch moves them into the slot (a block that starts late must still find the old ones).
// Tokens are staged a tile at a time in shared memory, the next tile travelling by cp.async while
// this one is worked; the per-token scalars (unit norms, beta, decays, gates) are made there in
// parallel, the running maximum by one lane in order.  The unit norms of q and k and dk^-1/2 are
// applied to the sums, not to the staged rows.  Everything is float32, and the order of every sum
// depends on the sizes alone, so a row's bits depend neither on the batch nor on how a prompt was cut.
#include "common.cuh"

namespace {

enum { MODE_DELTA = 0, MODE_GATED_SUM = 1 };
enum { GATE_SILU = 0, GATE_SIGMOID = 1 };
constexpr int VLANES = 16;               // virtual lanes of a column: the order of its sums is theirs

struct MatrixStateArgs {
    const float* q; const float* k; const float* v;      // [T, .] float32 rows
    int q_stride, k_stride, v_stride;
    const float* s0; const float* s1;                     // per (token, head) scalars: delta b, a; gated sum zi, zf
    int s0_stride, s1_stride;
    const float* c0; const float* c1;                     // per head constants: delta A_log, dt_bias; gated sum bi, bf
    float cap;
    const float* gate; int gate_stride;                   // [T, heads * dv] float32, or null
    int gate_act;
    const float* norm_weight; int norm_per_row;           // [dv], or [heads * dv] with norm_per_row
    float eps;
    const int* cu_q; const int* slots;
    float* state; long long state_stride;                 // floats per slot
    int heads, kv_heads, dk, dv;
    void* out; int out_bf16;                              // [T, heads * dv] in the activation dtype (fused epilogue)
    float* o_raw;                                         // [T, heads * dv] float32 (columns cut over blocks)
    float* carry;                                         // [requests, heads, dk + 1] float32 (columns cut, gated sum)
    int vec4;                                             // q, k, v rows and the heads in them start on 16 bytes
    int cut;                                              // a head's columns lie over several blocks
};

__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float gate_value(float g, int act) {
    const float s = 1.0f / (1.0f + expf(-g));
    return act == GATE_SILU ? g * s : s;
}

// Tokens a tile: two buffers of k and q rows and of v's columns (one is read while cp.async fills the
// other) and one of o must fit the 48 KB of static shared memory.
template <int DMAX, int CB> struct TileTokens {
    static constexpr int value = (4 * DMAX + 3 * (CB + 1)) * 16 * 4 <= 46 * 1024 ? 16 : 8;
};

// 4 bytes from global to shared memory behind the thread's back; zeros where `valid` is false
__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }

// The sum of a thread's VPT virtual lanes (neighbours first), then over the threads of a column.
template <int VPT, int LANES> __device__ __forceinline__ float lanes_sum(const float (&x)[VPT]) {
    float r = x[0];
    if (VPT == 4) r = (x[0] + x[1]) + (x[2] + x[3]);
#pragma unroll
    for (int sh = 1; sh < LANES; sh *= 2) r += __shfl_xor_sync(0xffffffffu, r, sh);
    return r;
}

// Small blocks of cut columns share an SM (the registers of at least 768 threads fit), so that other warps issue
// while one waits on its sums.
template <int MODE, int CB, int LANES> struct StateBlock {
    // columns a thread holds (a k or q read serves them all): two for the cut columns halved the warps that
    // hide one another's waits and was slower (2,048 tokens, 8 heads of 64 x 128: 460 -> 570 us)
    static constexpr int cpt = 1;
    static constexpr int threads = LANES * (CB / cpt) + (MODE == MODE_GATED_SUM ? 32 : 0);
    static constexpr int resident = LANES == 16 && 768 / threads > 0 ? 768 / threads : 1;
};

template <int MODE, int DMAX, int CB, int LANES>
__global__ void __launch_bounds__(StateBlock<MODE, CB, LANES>::threads, StateBlock<MODE, CB, LANES>::resident)
matrix_state_kernel(const MatrixStateArgs p) {
    constexpr int TT = TileTokens<DMAX, CB>::value;
    constexpr int VPT = VLANES / LANES;                   // virtual lanes a thread plays: 4 or 1
    constexpr int NG = DMAX / 64;                         // groups of 64 rows
    constexpr int NI = NG * VPT * 4;                      // state rows per thread
    constexpr int CS = CB + 1;                            // columns of o (the last: the normaliser's)
    constexpr int CPT = StateBlock<MODE, CB, LANES>::cpt;
    constexpr int GROUPS = CB / CPT;                      // threads along the columns
    constexpr int THREADS = StateBlock<MODE, CB, LANES>::threads;
    static_assert(DMAX % 64 == 0 && (VPT == 1 || VPT == 4) && THREADS >= 8 * TT && CB % 4 == 0 && CB % CPT == 0, "sizes");
    __shared__ __align__(16) float ks_[2][TT][DMAX];
    __shared__ __align__(16) float qs_[2][TT][DMAX];
    __shared__ __align__(16) float vs_[2][TT][CB];
    __shared__ float os[TT][CS];
    __shared__ float s0s[2][TT], s1s[2][TT];
    __shared__ float sa[TT], sb[TT], sfk[TT], sfq[TT], sm[TT], inv_s[TT], m_carry;
    const int req = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int c0 = blockIdx.z * CB;
    const int jc = tid / LANES, part = tid % LANES;       // column group of this block, share of its rows
    const int dk = p.dk, dv = p.dv;
    const int cols = dv + (MODE == MODE_GATED_SUM ? 1 : 0);              // columns of the stored state
    const bool is_norm_col = MODE == MODE_GATED_SUM && jc == GROUPS;     // its first column is the normaliser's
    int j[CPT];                                           // columns of the state
    bool live[CPT];
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
        j[cc] = is_norm_col ? dv : c0 + jc * CPT + cc;
        live[cc] = is_norm_col ? cc == 0 : (jc < GROUPS && j[cc] < dv);
    }
    const int t0 = p.cu_q[req], t1 = p.cu_q[req + 1];
    if (t0 >= t1) return;
    const int kvh = head / (p.heads / p.kv_heads);
    float* slot = p.state + (size_t)p.slots[req] * p.state_stride;
    float* s_head = slot + (size_t)head * dk * cols;
    float* m_state = slot + (size_t)p.heads * dk * cols + head;
    const bool fused = !p.cut;
    const float q_scale = rsqrtf((float)dk);
    const int row0 = part * (4 * VPT);                    // register ii holds row 64 (ii / (4 VPT)) + row0 + ii % (4 VPT)

    float S[CPT][NI];
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
        const int i = (ii / (4 * VPT)) * 64 + row0 + ii % (4 * VPT);
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) S[cc][ii] = (live[cc] && i < dk) ? s_head[(size_t)i * cols + j[cc]] : 0.0f;
    }
    if (MODE == MODE_GATED_SUM && tid == 0) m_carry = *m_state;

    // a tile's k, q, v and per-token scalars on their way into buffer `buf` (zeros outside the tile and the head)
    auto stage = [&](int buf, int tile0) {
        const int nt = min(TT, t1 - tile0);
        const float* kp = p.k + (size_t)kvh * dk;
        const float* qp = p.q + (size_t)kvh * dk;
        const float* vp = p.v + (size_t)head * dv + c0;
        if (p.vec4) {
            for (int e = tid; e < TT * (DMAX / 4); e += THREADS) {
                const int tt = e / (DMAX / 4), c = (e % (DMAX / 4)) * 4;
                const bool ok = tt < nt && c < dk;
                const size_t t = ok ? tile0 + tt : t0;
                cp_async16(&ks_[buf][tt][c], kp + t * p.k_stride + (ok ? c : 0), ok);
                cp_async16(&qs_[buf][tt][c], qp + t * p.q_stride + (ok ? c : 0), ok);
            }
            for (int e = tid; e < TT * (CB / 4); e += THREADS) {
                const int tt = e / (CB / 4), c = (e % (CB / 4)) * 4;
                const bool ok = tt < nt && c0 + c < dv;
                cp_async16(&vs_[buf][tt][c], vp + (size_t)(ok ? tile0 + tt : t0) * p.v_stride + (ok ? c : 0), ok);
            }
        } else {
            for (int e = tid; e < TT * DMAX; e += THREADS) {
                const int tt = e / DMAX, c = e % DMAX;
                const bool ok = tt < nt && c < dk;
                const size_t t = ok ? tile0 + tt : t0;
                cp_async4(&ks_[buf][tt][c], kp + t * p.k_stride + (ok ? c : 0), ok);
                cp_async4(&qs_[buf][tt][c], qp + t * p.q_stride + (ok ? c : 0), ok);
            }
            for (int e = tid; e < TT * CB; e += THREADS) {
                const int tt = e / CB, c = e % CB;
                const bool ok = tt < nt && c0 + c < dv;
                cp_async4(&vs_[buf][tt][c], vp + (size_t)(ok ? tile0 + tt : t0) * p.v_stride + (ok ? c : 0), ok);
            }
        }
        if (tid < TT) {
            const bool ok = tid < nt;
            const size_t t = ok ? tile0 + tid : t0;
            cp_async4(&s0s[buf][tid], p.s0 + t * p.s0_stride + head, ok);
            cp_async4(&s1s[buf][tid], p.s1 + t * p.s1_stride + head, ok);
        }
        cp_async_commit();
    };
    stage(0, t0);

    int buf = 0;
    for (int tile0 = t0; tile0 < t1; tile0 += TT, buf ^= 1) {
        const int nt = min(TT, t1 - tile0);
        float (*ks)[DMAX] = ks_[buf], (*qs)[DMAX] = qs_[buf];
        float (*vs)[CB] = vs_[buf];
        const float* s0t = s0s[buf];
        const float* s1t = s1s[buf];
        cp_async_wait_all();
        __syncthreads();                                  // this tile is in; the tile before is written out
        if (tile0 + TT < t1) stage(buf ^ 1, tile0 + TT);  // the next tile travels while this one is worked
        // ---- per-token scalars; past the portion's end a token that changes nothing (decay 1, write 0) ----
        if (MODE == MODE_DELTA) {
            if (tid < 8 * TT) {                           // eight lanes a token: the unit norms of q and k
                const int tt = tid / 8, l = tid % 8;
                float sq = 0.0f, sk = 0.0f;
                for (int c = l; c < DMAX; c += 8) {
                    sq = fmaf(qs[tt][c], qs[tt][c], sq);
                    sk = fmaf(ks[tt][c], ks[tt][c], sk);
                }
#pragma unroll
                for (int sh = 1; sh < 8; sh *= 2) {
                    sq += __shfl_xor_sync(0xffffffffu, sq, sh);
                    sk += __shfl_xor_sync(0xffffffffu, sk, sh);
                }
                if (l == 0) {
                    const bool in = tt < nt;
                    sfq[tt] = in ? q_scale / sqrtf(sq + 1e-6f) : 0.0f;
                    sfk[tt] = in ? 1.0f / sqrtf(sk + 1e-6f) : 0.0f;
                    sb[tt] = in ? 1.0f / (1.0f + expf(-s0t[tt])) : 0.0f;
                    sa[tt] = in ? expf(-expf(p.c0[head]) * softplusf_(s1t[tt] + p.c1[head])) : 1.0f;
                }
            }
        } else {
            if (tid < 32) {
                const int tt = tid;
                float gi = 0.0f, gf = 0.0f;
                if (tt < nt) {
                    gi = p.cap * tanhf((s0t[tt] + p.c0[head]) / p.cap);
                    gf = logsigmoidf_(p.cap * tanhf((s1t[tt] + p.c1[head]) / p.cap));
                }
                // the running maximum, in order: every lane walks the tile's gates in registers and keeps its own token's
                float m = m_carry, m_before = 0.0f, m_mine = 0.0f;
#pragma unroll
                for (int x = 0; x < TT; ++x) {
                    const float fx = __shfl_sync(0xffffffffu, gf, x), ix = __shfl_sync(0xffffffffu, gi, x);
                    if (x < nt) {
                        const float mn = fmaxf(fx + m, ix);
                        if (x == tt) { m_before = m; m_mine = mn; }
                        m = mn;
                    }
                }
                __syncwarp();
                if (tid == 0) m_carry = m;
                if (tt < TT) {
                    sm[tt] = tt < nt ? expf(-m_mine) : 1.0f;                    // what the normaliser is held against
                    sa[tt] = tt < nt ? expf(gf + m_before - m_mine) : 1.0f;
                    sb[tt] = tt < nt ? expf(gi - m_mine) : 0.0f;
                }
            }
        }
        __syncthreads();
        // ---- the recurrence: the tile's tokens one after another, no barrier between them -------
        float o_part[TT][CPT];
        auto token = [&](const int tt) {
            const float* krow = &ks[tt][row0];
            const float* qrow = &qs[tt][row0];
            const float dec = sa[tt];
            float vj[CPT], acc[CPT][VPT][4], w[VPT];
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc) vj[cc] = is_norm_col ? 1.0f : vs[tt][jc < GROUPS ? jc * CPT + cc : 0];
            if (MODE == MODE_DELTA) {
                const float fk = sfk[tt];
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc)
#pragma unroll
                    for (int v = 0; v < VPT; ++v) acc[cc][v][0] = acc[cc][v][1] = acc[cc][v][2] = acc[cc][v][3] = 0.0f;
#pragma unroll
                for (int g = 0; g < NG; ++g) {
#pragma unroll
                    for (int v = 0; v < VPT; ++v) {
                        const float4 kq = *reinterpret_cast<const float4*>(krow + g * 64 + v * 4);
                        const int at = (g * VPT + v) * 4;
#pragma unroll
                        for (int cc = 0; cc < CPT; ++cc) {
                            acc[cc][v][0] = fmaf(S[cc][at + 0], kq.x, acc[cc][v][0]);
                            acc[cc][v][1] = fmaf(S[cc][at + 1], kq.y, acc[cc][v][1]);
                            acc[cc][v][2] = fmaf(S[cc][at + 2], kq.z, acc[cc][v][2]);
                            acc[cc][v][3] = fmaf(S[cc][at + 3], kq.w, acc[cc][v][3]);
                        }
                    }
                }
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc) {
#pragma unroll
                    for (int v = 0; v < VPT; ++v)
                        w[v] = (acc[cc][v][0] + acc[cc][v][1]) + (acc[cc][v][2] + acc[cc][v][3]);
                    const float dot = fk * lanes_sum<VPT, LANES>(w);          // S^T k of the unit key
                    vj[cc] = fk * (sb[tt] * (vj[cc] - dec * dot));             // u, with the key's unit norm
                }
            } else {
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc) vj[cc] *= sb[tt];             // the input gate
            }
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc)
#pragma unroll
                for (int v = 0; v < VPT; ++v) acc[cc][v][0] = acc[cc][v][1] = acc[cc][v][2] = acc[cc][v][3] = 0.0f;
#pragma unroll
            for (int g = 0; g < NG; ++g) {
#pragma unroll
                for (int v = 0; v < VPT; ++v) {
                    const float4 kq = *reinterpret_cast<const float4*>(krow + g * 64 + v * 4);
                    const float4 qq = *reinterpret_cast<const float4*>(qrow + g * 64 + v * 4);
                    const int at = (g * VPT + v) * 4;
#pragma unroll
                    for (int cc = 0; cc < CPT; ++cc) {
                        S[cc][at + 0] = fmaf(dec, S[cc][at + 0], kq.x * vj[cc]);
                        S[cc][at + 1] = fmaf(dec, S[cc][at + 1], kq.y * vj[cc]);
                        S[cc][at + 2] = fmaf(dec, S[cc][at + 2], kq.z * vj[cc]);
                        S[cc][at + 3] = fmaf(dec, S[cc][at + 3], kq.w * vj[cc]);
                        acc[cc][v][0] = fmaf(S[cc][at + 0], qq.x, acc[cc][v][0]);
                        acc[cc][v][1] = fmaf(S[cc][at + 1], qq.y, acc[cc][v][1]);
                        acc[cc][v][2] = fmaf(S[cc][at + 2], qq.z, acc[cc][v][2]);
                        acc[cc][v][3] = fmaf(S[cc][at + 3], qq.w, acc[cc][v][3]);
                    }
                }
            }
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc) {
#pragma unroll
                for (int v = 0; v < VPT; ++v) w[v] = (acc[cc][v][0] + acc[cc][v][1]) + (acc[cc][v][2] + acc[cc][v][3]);
                o_part[tt][cc] = VPT == 4 ? (w[0] + w[VPT > 1 ? 1 : 0]) + (w[VPT > 2 ? 2 : 0] + w[VPT > 3 ? 3 : 0]) : w[0];
            }
        };
        if (nt == TT) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) token(tt);
        } else {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc) o_part[tt][cc] = 0.0f;
                if (tt < nt) token(tt);
            }
        }
#pragma unroll
        for (int sh = 1; sh < LANES; sh *= 2) {           // the threads of a column, all tokens of the tile at once
#pragma unroll
            for (int tt = 0; tt < TT; ++tt)
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc) o_part[tt][cc] += __shfl_xor_sync(0xffffffffu, o_part[tt][cc], sh);
        }
        if (part == 0 && (jc < GROUPS || is_norm_col)) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                const float scale = MODE == MODE_DELTA ? sfq[tt] : q_scale;
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc)
                    if (tt < nt && (!is_norm_col || cc == 0))
                        os[tt][is_norm_col ? CB : jc * CPT + cc] = live[cc] ? o_part[tt][cc] * scale : 0.0f;
            }
        }
        __syncthreads();
        if (MODE == MODE_GATED_SUM) {                     // the normaliser: n . q against e^-m
            for (int e = tid; e < nt * CB; e += THREADS) {
                const int tt = e / CB, c = e % CB;
                const float den = fmaxf(fabsf(os[tt][CB]), sm[tt]) + 1e-6f;
                os[tt][c] = os[tt][c] / den;
            }
            __syncthreads();
        }
        if (!fused) {
            for (int e = tid; e < nt * CB; e += THREADS) {
                const int tt = e / CB, c = c0 + e % CB;
                if (c < dv) p.o_raw[(size_t)(tile0 + tt) * p.heads * dv + head * dv + c] = os[tt][e % CB];
            }
            continue;
        }
        for (int tt = tid / 32; tt < nt; tt += THREADS / 32) {       // a warp per token: its unit norm
            float ss = 0.0f;
            for (int c = tid % 32; c < dv; c += 32) ss = fmaf(os[tt][c], os[tt][c], ss);
            ss = warp_sum(ss);
            if (tid % 32 == 0) inv_s[tt] = 1.0f / sqrtf(ss / (float)dv + p.eps);
        }
        __syncthreads();
        for (int e = tid; e < nt * CB; e += THREADS) {
            const int tt = e / CB, c = e % CB;
            if (c < dv) {
                const size_t t = tile0 + tt;
                float y = os[tt][c] * inv_s[tt] * p.norm_weight[(p.norm_per_row ? head * dv : 0) + c];
                if (p.gate) y *= gate_value(p.gate[t * p.gate_stride + head * dv + c], p.gate_act);
                const size_t at = t * p.heads * dv + head * dv + c;
                if (p.out_bf16) ((bf16*)p.out)[at] = __float2bfloat16_rn(y);
                else ((float*)p.out)[at] = y;
            }
        }
    }
    __syncthreads();
    float* carry = fused ? nullptr : p.carry + ((size_t)req * p.heads + head) * (dk + 1);
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
        if (live[cc] && (!is_norm_col || blockIdx.z == 0)) {
#pragma unroll
            for (int ii = 0; ii < NI; ++ii) {
                const int i = (ii / (4 * VPT)) * 64 + row0 + ii % (4 * VPT);
                if (i < dk) {
                    if (is_norm_col && !fused) carry[i] = S[cc][ii];
                    else s_head[(size_t)i * cols + j[cc]] = S[cc][ii];
                }
            }
        }
    }
    if (MODE == MODE_GATED_SUM && tid == 0 && blockIdx.z == 0) {
        if (fused) *m_state = m_carry;
        else carry[dk] = m_carry;
    }
}

// The gated sum's normaliser column and running maximum from `carry` into the slots, after every
// block of the cut launch has read the old ones: one block per (request, head).
__global__ void __launch_bounds__(64)
matrix_state_commit_kernel(const float* __restrict__ carry, const int* __restrict__ cu_q,
                           const int* __restrict__ slots, float* state, long long state_stride, int heads, int dk,
                           int dv) {
    const int req = blockIdx.x, head = blockIdx.y;
    if (cu_q[req] >= cu_q[req + 1]) return;
    const int cols = dv + 1;
    const float* c = carry + ((size_t)req * heads + head) * (dk + 1);
    float* slot = state + (size_t)slots[req] * state_stride;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) slot[((size_t)head * dk + i) * cols + dv] = c[i];
    if (threadIdx.x == 0) slot[(size_t)heads * dk * cols + head] = c[dk];
}

// out[t, head] = o / rms(o) * weight * act(gate) for rows that column-cut blocks left as float32:
// one warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(256)
matrix_state_finish_kernel(const float* o_raw, const float* __restrict__ norm_weight, int norm_per_row, float eps,
                           const float* gate, int gate_stride, int gate_act, int rows, int heads, int dv,
                           TO* __restrict__ out) {
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= rows * heads) return;
    const int t = unit / heads, head = unit % heads;
    const float* o = o_raw + (size_t)unit * dv;
    float ss = 0.0f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(o[c], o[c], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        float y = o[c] * inv * norm_weight[(norm_per_row ? head * dv : 0) + c];
        if (gate) y *= gate_value(gate[(size_t)t * gate_stride + head * dv + c], gate_act);
        out[(size_t)unit * dv + c] = from_f32<TO>(y);
    }
}

template <int MODE, int DMAX>
int launch_cb(const MatrixStateArgs& a, int requests, int cb, int col_blocks, cudaStream_t s) {
    dim3 grid(requests, a.heads, col_blocks);
#define TI_MS_GO(CB_, LANES_) \
    matrix_state_kernel<MODE, DMAX, CB_, LANES_><<<grid, StateBlock<MODE, CB_, LANES_>::threads, 0, s>>>(a)
    if (a.cut && cb == 8) TI_MS_GO(8, 16);
    else if (a.cut && cb == 16) TI_MS_GO(16, 16);
    else if (a.cut && cb == 32) TI_MS_GO(32, 16);
    else if (cb == 32) TI_MS_GO(32, 4);
    else if (cb == 64) TI_MS_GO(64, 4);
    else TI_MS_GO(128, 4);
#undef TI_MS_GO
    return 0;
}

template <int MODE>
int launch_dk(const MatrixStateArgs& a, int requests, int cb, int col_blocks, cudaStream_t s) {
    if (a.dk <= 64) return launch_cb<MODE, 64>(a, requests, cb, col_blocks, s);
    if (a.dk <= 128) return launch_cb<MODE, 128>(a, requests, cb, col_blocks, s);
    return launch_cb<MODE, 256>(a, requests, cb, col_blocks, s);
}

}  // namespace

// Floats of state per request: every head's S (with the normaliser's column in the gated sum) and,
// in the gated sum, one running maximum per head.
extern "C" long long ti_matrix_state_floats(int mode, int heads, int dk, int dv) {
    return mode == MODE_GATED_SUM ? (long long)heads * dk * (dv + 1) + heads : (long long)heads * dk * dv;
}

// col_block: 0 = a head's columns in one block (dv <= 128) with the norm, weight and gate in the same launch;
// 8, 16, 32, 64 or 128 = that many columns a block (16 threads a column up to 32 columns, 4 beyond), o left in
// `o_raw` and finished by a second launch.
extern "C" int ti_matrix_state(int mode, const float* q, const float* k, const float* v, int q_stride, int k_stride,
                               int v_stride, const float* s0, int s0_stride, const float* s1, int s1_stride,
                               const float* c0, const float* c1, float cap, const float* gate, int gate_stride,
                               int gate_act, const float* norm_weight, int norm_per_row, float eps,
                               const int* cu_q, const int* slots, int requests, int rows, float* state,
                               long long state_stride, int heads, int kv_heads, int dk, int dv, int col_block,
                               void* out, int out_dtype, float* o_raw, float* carry, void* stream) {
    if (requests == 0 || rows == 0) return 0;
    TI_REQUIRE(mode == MODE_DELTA || mode == MODE_GATED_SUM, "matrix_state: mode %d", mode);
    TI_REQUIRE(dk >= 1 && dk <= 256 && dv >= 1 && dv <= 1024, "matrix_state: head sizes %d x %d (keys up to 256, "
               "values up to 1,024)", dk, dv);
    TI_REQUIRE(heads >= 1 && kv_heads >= 1 && heads % kv_heads == 0, "matrix_state: %d heads over %d key heads",
               heads, kv_heads);
    TI_REQUIRE(out_dtype == TI_F32 || out_dtype == TI_BF16, "matrix_state: output dtype code %d", out_dtype);
    TI_REQUIRE(col_block == 0 || col_block == 8 || col_block == 16 || col_block == 32 || col_block == 64 || col_block == 128,
               "matrix_state: %d columns a block", col_block);
    TI_REQUIRE(col_block != 0 || dv <= 128, "matrix_state: %d value columns do not fit one block", dv);
    TI_REQUIRE(col_block == 0 || o_raw != nullptr, "matrix_state: cut columns need the float32 rows");
    TI_REQUIRE(col_block == 0 || mode != MODE_GATED_SUM || carry != nullptr,
               "matrix_state: cut columns of the gated sum need room for the normaliser and the maximum");
    MatrixStateArgs a;
    a.q = q; a.k = k; a.v = v; a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
    a.s0 = s0; a.s1 = s1; a.s0_stride = s0_stride; a.s1_stride = s1_stride; a.c0 = c0; a.c1 = c1; a.cap = cap;
    a.gate = gate; a.gate_stride = gate_stride; a.gate_act = gate_act;
    a.norm_weight = norm_weight; a.norm_per_row = norm_per_row; a.eps = eps;
    a.cu_q = cu_q; a.slots = slots; a.state = state; a.state_stride = state_stride;
    a.heads = heads; a.kv_heads = kv_heads; a.dk = dk; a.dv = dv;
    a.out = out; a.out_bf16 = out_dtype == TI_BF16; a.o_raw = o_raw; a.carry = carry;
    a.cut = col_block != 0;
    a.vec4 = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) % 16 == 0 &&
              q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 && dk % 4 == 0 && dv % 4 == 0) ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    int cb = col_block, col_blocks = 1;
    if (cb == 0) cb = dv <= 32 ? 32 : dv <= 64 ? 64 : 128;
    else col_blocks = (dv + cb - 1) / cb;
    if (mode == MODE_DELTA) launch_dk<MODE_DELTA>(a, requests, cb, col_blocks, s);
    else launch_dk<MODE_GATED_SUM>(a, requests, cb, col_blocks, s);
    if (int rc = ti_check_launch("matrix_state")) return rc;
    if (col_block != 0) {
        if (mode == MODE_GATED_SUM) {
            matrix_state_commit_kernel<<<dim3(requests, heads), 64, 0, s>>>(carry, cu_q, slots, state, state_stride,
                                                                            heads, dk, dv);
            if (int rc = ti_check_launch("matrix_state_commit")) return rc;
        }
        const int blocks = (rows * heads + 7) / 8;
        if (out_dtype == TI_BF16)
            matrix_state_finish_kernel<bf16><<<blocks, 256, 0, s>>>(o_raw, norm_weight, norm_per_row, eps, gate,
                                                                     gate_stride, gate_act, rows, heads, dv, (bf16*)out);
        else
            matrix_state_finish_kernel<float><<<blocks, 256, 0, s>>>(o_raw, norm_weight, norm_per_row, eps, gate,
                                                                      gate_stride, gate_act, rows, heads, dv, (float*)out);
        return ti_check_launch("matrix_state_finish");
    }
    return 0;
}
