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
// One block walks the tokens of one (request, head) in order.  A column of S belongs to four
// neighbouring lanes, each holding a quarter of its rows in registers; a head's columns may be
// cut over several blocks (few requests with long portions), which then write o as float32 and
// leave the norm, the weight and the gate to `matrix_state_finish`.  In the gated sum every such
// block reads the normaliser's column and the running maximum, so their new values wait in
// `carry` until all blocks are through and a small launch moves them into the slot (a block that
// starts late must still find the old ones).  Tokens are staged a tile at a
// time in shared memory; the per-token scalars (unit norms, beta, decays, gates) are made there
// in parallel, the running maximum by one lane in order.  Everything is float32, and the order
// of every sum depends on the sizes alone, so a row's bits depend neither on the batch nor on
// how a prompt was cut.
#include "common.cuh"

namespace {

enum { MODE_DELTA = 0, MODE_GATED_SUM = 1 };
enum { GATE_SILU = 0, GATE_SIGMOID = 1 };
constexpr int LANES = 4;

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
};

__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float gate_value(float g, int act) {
    const float s = 1.0f / (1.0f + expf(-g));
    return act == GATE_SILU ? g * s : s;
}

template <int DMAX, int CB> struct TileTokens {
    static constexpr int value = (2 * DMAX + 2 * (CB + 1)) * 16 * 4 <= 40 * 1024 ? 16 : 8;
};

template <int MODE, int DMAX, int CB>
__global__ void __launch_bounds__(LANES * CB + (MODE == MODE_GATED_SUM ? 32 : 0))
matrix_state_kernel(const MatrixStateArgs p) {
    constexpr int TT = TileTokens<DMAX, CB>::value;
    constexpr int NI = DMAX / LANES;                      // state rows per thread
    constexpr int CS = CB + 1;                            // staged columns (the last: the normaliser's value 1)
    constexpr int THREADS = LANES * CB + (MODE == MODE_GATED_SUM ? 32 : 0);
    __shared__ __align__(16) float ks[TT][DMAX], qs[TT][DMAX];
    __shared__ float vs[TT][CS], os[TT][CS];
    __shared__ float sa[TT], sb[TT], sm[TT], inv_s[TT], m_carry;
    const int req = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int c0 = blockIdx.z * CB;
    const int jc = tid / LANES, part = tid % LANES;       // column of this block, quarter of its rows
    const int dk = p.dk, dv = p.dv;
    const int cols = dv + (MODE == MODE_GATED_SUM ? 1 : 0);              // columns of the stored state
    const bool is_norm_col = MODE == MODE_GATED_SUM && jc == CB;
    const int j = is_norm_col ? dv : c0 + jc;             // column of the state
    const bool live = is_norm_col ? part < LANES : (jc < CB && j < dv);
    const int t0 = p.cu_q[req], t1 = p.cu_q[req + 1];
    if (t0 >= t1) return;
    const int kvh = head / (p.heads / p.kv_heads);
    float* slot = p.state + (size_t)p.slots[req] * p.state_stride;
    float* s_head = slot + (size_t)head * dk * cols;
    float* m_state = slot + (size_t)p.heads * dk * cols + head;
    const bool fused = gridDim.z == 1;
    const float q_scale = rsqrtf((float)dk);

    // lane `part` of a column holds rows 16 g + 4 part + x (x = 0..3): the lanes of a column read
    // neighbouring 16-byte pieces of a token's k and q
    float S[NI];
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
        const int i = (ii / 4) * (4 * LANES) + part * 4 + ii % 4;
        S[ii] = (live && i < dk) ? s_head[(size_t)i * cols + j] : 0.0f;
    }
    if (MODE == MODE_GATED_SUM && tid == 0) m_carry = *m_state;

    for (int tile0 = t0; tile0 < t1; tile0 += TT) {
        const int nt = min(TT, t1 - tile0);
        __syncthreads();                                  // the tile before is written out
        for (int e = tid; e < TT * DMAX; e += THREADS) {
            const int tt = e / DMAX, c = e % DMAX;
            const bool ok = tt < nt && c < dk;
            ks[tt][c] = ok ? p.k[(size_t)(tile0 + tt) * p.k_stride + kvh * dk + c] : 0.0f;
            qs[tt][c] = ok ? p.q[(size_t)(tile0 + tt) * p.q_stride + kvh * dk + c] : 0.0f;
        }
        for (int e = tid; e < TT * CS; e += THREADS) {
            const int tt = e / CS, c = e % CS;
            float x = 0.0f;
            if (c == CB) x = 1.0f;
            else if (tt < nt && c0 + c < dv) x = p.v[(size_t)(tile0 + tt) * p.v_stride + head * dv + c0 + c];
            vs[tt][c] = x;
        }
        __syncthreads();
        // ---- per-token scalars -----------------------------------------------------------------
        if (MODE == MODE_DELTA) {
            for (int tt = tid / 32; tt < nt; tt += THREADS / 32) {
                const int lane = tid % 32;
                float sq = 0.0f, sk = 0.0f;
                for (int c = lane; c < dk; c += 32) {
                    sq = fmaf(qs[tt][c], qs[tt][c], sq);
                    sk = fmaf(ks[tt][c], ks[tt][c], sk);
                }
                sq = warp_sum(sq);
                sk = warp_sum(sk);
                const float fq = q_scale / sqrtf(sq + 1e-6f), fk = 1.0f / sqrtf(sk + 1e-6f);
                for (int c = lane; c < dk; c += 32) { qs[tt][c] *= fq; ks[tt][c] *= fk; }
                if (lane == 0) {
                    const size_t t = tile0 + tt;
                    const float b = p.s0[t * p.s0_stride + head], a = p.s1[t * p.s1_stride + head];
                    sb[tt] = 1.0f / (1.0f + expf(-b));
                    sa[tt] = expf(-expf(p.c0[head]) * softplusf_(a + p.c1[head]));
                }
            }
        } else {
            if (tid < 32) {
                const int tt = tid;
                float gi = 0.0f, gf = 0.0f;
                if (tt < nt) {
                    const size_t t = tile0 + tt;
                    gi = p.cap * tanhf((p.s0[t * p.s0_stride + head] + p.c0[head]) / p.cap);
                    gf = logsigmoidf_(p.cap * tanhf((p.s1[t * p.s1_stride + head] + p.c1[head]) / p.cap));
                    sa[tt] = gf;
                    sb[tt] = gi;
                }
                __syncwarp();
                if (tid == 0) {                           // the running maximum, in order
                    float m = m_carry;
                    for (int x = 0; x < nt; ++x) {
                        const float mn = fmaxf(sa[x] + m, sb[x]);
                        inv_s[x] = m;                     // the maximum before this token
                        sm[x] = mn;
                        m = mn;
                    }
                    m_carry = m;
                }
                __syncwarp();
                if (tt < nt) {
                    sa[tt] = expf(gf + inv_s[tt] - sm[tt]);
                    sb[tt] = expf(gi - sm[tt]);
                }
            }
            __syncthreads();
            for (int e = tid; e < nt * DMAX; e += THREADS) {
                const int tt = e / DMAX, c = e % DMAX;
                ks[tt][c] *= sb[tt];                      // the input gate rides on the key
                qs[tt][c] *= q_scale;
            }
        }
        __syncthreads();
        // ---- the recurrence: the tile's tokens one after another, no barrier between them -------
        float o_part[TT];
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            o_part[tt] = 0.0f;
            if (tt < nt) {
                const float vj = vs[tt][is_norm_col ? CB : (jc < CB ? jc : 0)];
                const float4* k4 = reinterpret_cast<const float4*>(&ks[tt][part * 4]);
                const float4* q4 = reinterpret_cast<const float4*>(&qs[tt][part * 4]);
                const float dec = sa[tt];
                if (MODE == MODE_DELTA) {
                    float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
                    for (int g4 = 0; g4 < NI / 4; ++g4) {
                        const float4 kq = k4[g4 * LANES];
                        d0 = fmaf(S[g4 * 4 + 0], kq.x, d0);
                        d1 = fmaf(S[g4 * 4 + 1], kq.y, d1);
                        d2 = fmaf(S[g4 * 4 + 2], kq.z, d2);
                        d3 = fmaf(S[g4 * 4 + 3], kq.w, d3);
                    }
                    float dot = (d0 + d1) + (d2 + d3);
                    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                    const float u = sb[tt] * (vj - dec * dot);
                    float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
                    for (int g4 = 0; g4 < NI / 4; ++g4) {
                        const float4 kq = k4[g4 * LANES], qq = q4[g4 * LANES];
                        S[g4 * 4 + 0] = fmaf(dec, S[g4 * 4 + 0], kq.x * u);
                        S[g4 * 4 + 1] = fmaf(dec, S[g4 * 4 + 1], kq.y * u);
                        S[g4 * 4 + 2] = fmaf(dec, S[g4 * 4 + 2], kq.z * u);
                        S[g4 * 4 + 3] = fmaf(dec, S[g4 * 4 + 3], kq.w * u);
                        o0 = fmaf(S[g4 * 4 + 0], qq.x, o0);
                        o1 = fmaf(S[g4 * 4 + 1], qq.y, o1);
                        o2 = fmaf(S[g4 * 4 + 2], qq.z, o2);
                        o3 = fmaf(S[g4 * 4 + 3], qq.w, o3);
                    }
                    o_part[tt] = (o0 + o1) + (o2 + o3);
                } else {
                    float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
                    for (int g4 = 0; g4 < NI / 4; ++g4) {
                        const float4 kq = k4[g4 * LANES], qq = q4[g4 * LANES];
                        S[g4 * 4 + 0] = fmaf(dec, S[g4 * 4 + 0], kq.x * vj);
                        S[g4 * 4 + 1] = fmaf(dec, S[g4 * 4 + 1], kq.y * vj);
                        S[g4 * 4 + 2] = fmaf(dec, S[g4 * 4 + 2], kq.z * vj);
                        S[g4 * 4 + 3] = fmaf(dec, S[g4 * 4 + 3], kq.w * vj);
                        o0 = fmaf(S[g4 * 4 + 0], qq.x, o0);
                        o1 = fmaf(S[g4 * 4 + 1], qq.y, o1);
                        o2 = fmaf(S[g4 * 4 + 2], qq.z, o2);
                        o3 = fmaf(S[g4 * 4 + 3], qq.w, o3);
                    }
                    o_part[tt] = (o0 + o1) + (o2 + o3);
                }
            }
        }
#pragma unroll
        for (int sh = 1; sh < LANES; sh *= 2) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) o_part[tt] += __shfl_xor_sync(0xffffffffu, o_part[tt], sh);
        }
        if (part == 0 && (jc < CB || is_norm_col)) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt)
                if (tt < nt) os[tt][is_norm_col ? CB : jc] = live ? o_part[tt] : 0.0f;
        }
        __syncthreads();
        if (MODE == MODE_GATED_SUM) {                     // the normaliser: n . q against e^-m
            for (int e = tid; e < nt * CB; e += THREADS) {
                const int tt = e / CB, c = e % CB;
                const float den = fmaxf(fabsf(os[tt][CB]), expf(-sm[tt])) + 1e-6f;
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
    if (live && (!is_norm_col || blockIdx.z == 0)) {
#pragma unroll
        for (int ii = 0; ii < NI; ++ii) {
            const int i = (ii / 4) * (4 * LANES) + part * 4 + ii % 4;
            if (i < dk) {
                if (is_norm_col && !fused) carry[i] = S[ii];
                else s_head[(size_t)i * cols + j] = S[ii];
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
    const int extra = MODE == MODE_GATED_SUM ? 32 : 0;
    if (cb == 32) matrix_state_kernel<MODE, DMAX, 32><<<grid, LANES * 32 + extra, 0, s>>>(a);
    else if (cb == 64) matrix_state_kernel<MODE, DMAX, 64><<<grid, LANES * 64 + extra, 0, s>>>(a);
    else matrix_state_kernel<MODE, DMAX, 128><<<grid, LANES * 128 + extra, 0, s>>>(a);
    return 0;
}

template <int MODE>
int launch_dk(const MatrixStateArgs& a, int requests, int cb, int col_blocks, cudaStream_t s) {
    if (a.dk <= 32) return launch_cb<MODE, 32>(a, requests, cb, col_blocks, s);
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
// 32, 64 or 128 = that many columns a block, o left in `o_raw` and finished by a second launch.
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
    TI_REQUIRE(col_block == 0 || col_block == 32 || col_block == 64 || col_block == 128,
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
