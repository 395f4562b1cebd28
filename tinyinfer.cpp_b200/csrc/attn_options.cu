// Paged attention with optional parts, on the CUDA cores, and the kernels that prepare its heads.
//
//  * qk_rownorm_rope_store: from a float32 product with the columns [queries | keys | values |
//    anything else], norms the whole query row and the whole key row (RMS over all heads at once,
//    one weight per column), turns the first `rot` elements of every head by the token's position
//    (neighbouring elements 2i, 2i + 1 form a pair; angle = position * inv_freq[i]), writes keys
//    and values into the token's page and the queries out.
//  * latent_prepare: from a float32 product with the columns [query heads of (dk plain | dr
//    rotated) | latent of `rank` | one rotated key part of dr]: the latent is normed (RMS, a weight
//    per element) and stored with the turned key part as ONE row of the token's page; the plain
//    query parts and the turned query parts go out separately.
//  * qkv_turn_store: the same columns without any norm: the first `rot` elements of every query and key
//    head are turned by the token's position (pairs of neighbours, or element i with i + rot/2), the
//    first `v_rot` elements of every value head by frequencies of their own, keys and values go into
//    the token's page and the queries out.  turn_rows turns the heads of finished rows by plus or minus
//    their position (the way back for outputs over turned values) and multiplies by sigmoid(gate).
//  * slice_rmsnorm: the RMS norm (a weight per element) of the first n columns of rows with a stride.
//  * head_project: out[t, h, :] = in[t, h, :] W[h] with a matrix [n_in, n_out] per head.
//  * attention_options: one block per (token, query head).  Token i sees key j <= i when j is not
//    behind the window (i - j < window) and not in an earlier chunk (j >= floor(i / chunk) *
//    chunk); score = (q . k) * scale, times head_scale[h] if given, then cap * tanh(score / cap)
//    if cap > 0; softmax over the visible keys, whose denominator also counts exp(sink[h]) if a
//    sink is given; the normalised output is multiplied by sigmoid(gate), one gate per head or
//    one per output element.  With `shared_rows` a page holds one row of dk elements per token
//    and kv head, and the value of a key is the first dv elements of that row.
//
// All arithmetic is float32 (positions, angles, norms, scores, softmax weights, the weighted sum);
// inputs and outputs may be float32 or bfloat16.  The order in which a row's keys are added
// depends on the row alone, so a row's bits do not depend on the batch or on how a prompt was cut.
// Page layout without `shared_rows`: keys [kv head][slot][dk], behind them values [kv head][slot][dv].
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
enum { TI_ERR_BAD_PAGE = 1 };

__device__ __forceinline__ float turned(const float* x, int j, float pos, const float* inv_freq, float unit) {
    // element j (inside the rotated width) of a head x after the turn; `unit` scales both inputs
    float s, c;
    sincosf(pos * inv_freq[j >> 1], &s, &c);
    const float a = x[j] * unit, b = x[j ^ 1] * unit;
    return (j & 1) ? a * c + b * s : a * c - b * s;
}

// The turn of a head by a table of the token's cosines and sines (`cs[pair]`, made once per token: the angle
// depends on the position and the pair alone, not on the head).  A head of n elements whose first `rot` are
// turned has rot/2 pairs and n - rot single elements: item i < rot/2 is pair i, the others are singles.
struct TurnItem { int a, b; };      // the pair's two elements (b < 0: a single element a)
__device__ __forceinline__ TurnItem turn_item(int i, int rot, int halves) {
    const int half = rot >> 1;
    if (i >= half) return {rot + (i - half), -1};
    return halves ? TurnItem{i, i + half} : TurnItem{2 * i, 2 * i + 1};
}

__device__ __forceinline__ void fill_turn_table(float2* cs, int pairs, float pos, const float* __restrict__ inv_freq,
                                                float mag) {
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        cs[i] = make_float2(c * mag, s * mag);
    }
}

template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
qkv_turn_store_kernel(const float* proj, int stride, const float* __restrict__ inv_freq, int rot, int halves, float mag,
                      const float* __restrict__ v_inv_freq, int v_rot, int v_halves,
                      const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                      const int* __restrict__ block_table, int bt_stride, TC* __restrict__ pages, int num_pages,
                      int page_size, int write_kv, int num_heads, int num_kv_heads, int dk, int dv,
                      TQ* __restrict__ q_out, int* __restrict__ status) {
    extern __shared__ float2 turn_table[];             // rot/2 entries for queries and keys, then v_rot/2 for values
    const int t = blockIdx.x;
    const int nq = num_heads * dk, nk = num_kv_heads * dk;
    const float* row = proj + (size_t)t * stride;
    const int pos_i = positions[t];
    const float pos = (float)pos_i;
    float2* cs = turn_table;
    float2* vcs = turn_table + (rot >> 1);
    fill_turn_table(cs, rot >> 1, pos, inv_freq, mag);
    if (write_kv) fill_turn_table(vcs, v_rot >> 1, pos, v_inv_freq, 1.0f);
    __syncthreads();
    const int per_head = (rot >> 1) + (dk - rot);      // items of a query or key head
    for (int e = threadIdx.x; e < num_heads * per_head; e += blockDim.x) {
        const int h = e / per_head, i = e % per_head;
        const TurnItem it = turn_item(i, rot, halves);
        const float* x = row + (size_t)h * dk;
        TQ* dst = q_out + (size_t)t * nq + (size_t)h * dk;
        if (it.b < 0) { dst[it.a] = from_f32<TQ>(x[it.a]); continue; }
        const float2 f = cs[i];
        dst[it.a] = from_f32<TQ>(x[it.a] * f.x - x[it.b] * f.y);
        dst[it.b] = from_f32<TQ>(x[it.b] * f.x + x[it.a] * f.y);
    }
    if (!write_kv) return;
    const int page = block_table[(size_t)req_of_tok[t] * bt_stride + pos_i / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
        return;
    }
    const int slot = pos_i % page_size;
    TC* base = pages + (size_t)page * num_kv_heads * page_size * (dk + dv);
    const float* krow = row + nq;
    for (int e = threadIdx.x; e < num_kv_heads * per_head; e += blockDim.x) {
        const int g = e / per_head, i = e % per_head;
        const TurnItem it = turn_item(i, rot, halves);
        const float* x = krow + (size_t)g * dk;
        TC* dst = base + ((size_t)g * page_size + slot) * dk;
        if (it.b < 0) { dst[it.a] = from_f32<TC>(x[it.a]); continue; }
        const float2 f = cs[i];
        dst[it.a] = from_f32<TC>(x[it.a] * f.x - x[it.b] * f.y);
        dst[it.b] = from_f32<TC>(x[it.b] * f.x + x[it.a] * f.y);
    }
    TC* vbase = base + (size_t)num_kv_heads * page_size * dk;
    const float* vrow = krow + nk;
    const int v_per_head = (v_rot >> 1) + (dv - v_rot);
    for (int e = threadIdx.x; e < num_kv_heads * v_per_head; e += blockDim.x) {
        const int g = e / v_per_head, i = e % v_per_head;
        const TurnItem it = turn_item(i, v_rot, v_halves);
        const float* x = vrow + (size_t)g * dv;
        TC* dst = vbase + ((size_t)g * page_size + slot) * dv;
        if (it.b < 0) { dst[it.a] = from_f32<TC>(x[it.a]); continue; }
        const float2 f = vcs[i];
        dst[it.a] = from_f32<TC>(x[it.a] * f.x - x[it.b] * f.y);
        dst[it.b] = from_f32<TC>(x[it.b] * f.x + x[it.a] * f.y);
    }
}

// x[t, h, :] turned by sign * position over its first `rot` elements, then times sigmoid(gate[t, h * n + j]); a
// block per token, a thread reads and writes both elements of a pair, so the rows may be turned in place
template <typename T>
__global__ void __launch_bounds__(256)
turn_rows_kernel(const T* x, const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot,
                 int halves, float sign, const float* gate, int gate_stride, int num_heads, int n, T* out) {
    extern __shared__ float2 turn_table[];
    const int t = blockIdx.x;
    fill_turn_table(turn_table, rot >> 1, sign * (float)positions[t], inv_freq, 1.0f);
    __syncthreads();
    const int per_head = (rot >> 1) + (n - rot);
    const float* gt = gate ? gate + (size_t)t * gate_stride : nullptr;
    for (int e = threadIdx.x; e < num_heads * per_head; e += blockDim.x) {
        const int h = e / per_head, i = e % per_head;
        const TurnItem it = turn_item(i, rot, halves);
        const size_t at = ((size_t)t * num_heads + h) * n;
        const float a = to_f32(x[at + it.a]);
        if (it.b < 0) {
            out[at + it.a] = from_f32<T>(gt ? a / (1.0f + expf(-gt[(size_t)h * n + it.a])) : a);
            continue;
        }
        const float b = to_f32(x[at + it.b]);
        const float2 f = turn_table[i];
        float ya = a * f.x - b * f.y, yb = b * f.x + a * f.y;
        if (gt) {
            ya *= 1.0f / (1.0f + expf(-gt[(size_t)h * n + it.a]));
            yb *= 1.0f / (1.0f + expf(-gt[(size_t)h * n + it.b]));
        }
        out[at + it.a] = from_f32<T>(ya);
        out[at + it.b] = from_f32<T>(yb);
    }
}

template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
qk_rownorm_rope_store_kernel(const float* proj, int stride, const float* __restrict__ q_weight,
                             const float* __restrict__ k_weight, float eps,
                             const float* __restrict__ inv_freq, int rot,
                             const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                             const int* __restrict__ block_table, int bt_stride, TC* __restrict__ pages,
                             int num_pages, int page_size, int write_kv, int num_heads, int num_kv_heads,
                             int dk, int dv, TQ* __restrict__ q_out, int* __restrict__ status) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int nq = num_heads * dk, nk = num_kv_heads * dk, nv = num_kv_heads * dv;
    const float* row = proj + (size_t)t * stride;
    const int pos_i = positions[t];
    const float pos = (float)pos_i;
    float ss = 0.0f;
    for (int e = threadIdx.x; e < nq; e += blockDim.x) ss = fmaf(row[e], row[e], ss);
    const float inv_q = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nq + eps);
    for (int e = threadIdx.x; e < nq; e += blockDim.x) {
        const int j = e % dk;
        const float* head = row + (e - j);
        const float* w = q_weight ? q_weight + (e - j) : nullptr;
        float y;
        if (j < rot) {
            // the weight belongs to the element, so it is applied before the turn
            float s, c;
            sincosf(pos * inv_freq[j >> 1], &s, &c);
            const float a = head[j] * inv_q * (w ? w[j] : 1.0f);
            const float b = head[j ^ 1] * inv_q * (w ? w[j ^ 1] : 1.0f);
            y = (j & 1) ? a * c + b * s : a * c - b * s;
        } else {
            y = head[j] * inv_q * (w ? w[j] : 1.0f);
        }
        q_out[(size_t)t * nq + e] = from_f32<TQ>(y);
    }
    if (!write_kv) return;
    const int page = block_table[(size_t)req_of_tok[t] * bt_stride + pos_i / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
        return;
    }
    const int slot = pos_i % page_size;
    TC* base = pages + (size_t)page * num_kv_heads * page_size * (dk + dv);
    const float* krow = row + nq;
    ss = 0.0f;
    for (int e = threadIdx.x; e < nk; e += blockDim.x) ss = fmaf(krow[e], krow[e], ss);
    const float inv_k = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nk + eps);
    for (int e = threadIdx.x; e < nk; e += blockDim.x) {
        const int j = e % dk, g = e / dk;
        const float* head = krow + (e - j);
        const float* w = k_weight ? k_weight + (e - j) : nullptr;
        float y;
        if (j < rot) {
            float s, c;
            sincosf(pos * inv_freq[j >> 1], &s, &c);
            const float a = head[j] * inv_k * (w ? w[j] : 1.0f);
            const float b = head[j ^ 1] * inv_k * (w ? w[j ^ 1] : 1.0f);
            y = (j & 1) ? a * c + b * s : a * c - b * s;
        } else {
            y = head[j] * inv_k * (w ? w[j] : 1.0f);
        }
        base[((size_t)g * page_size + slot) * dk + j] = from_f32<TC>(y);
    }
    TC* vbase = base + (size_t)num_kv_heads * page_size * dk;
    const float* vrow = krow + nk;
    for (int e = threadIdx.x; e < nv; e += blockDim.x) {
        const int j = e % dv, g = e / dv;
        vbase[((size_t)g * page_size + slot) * dv + j] = from_f32<TC>(vrow[e]);
    }
}

// out[t, :] = x[t, :n] / sqrt(mean(x[t, :n]^2) + eps) * w over rows with a stride: the norm of a column slice of a
// product (a latent that shares its product with other columns)
template <typename TO>
__global__ void __launch_bounds__(256)
slice_rmsnorm_kernel(const float* x, int stride, int n, const float* __restrict__ w, float eps, TO* __restrict__ out) {
    __shared__ float scratch[32];
    const float* row = x + (size_t)blockIdx.x * stride;
    float ss = 0.0f;
    for (int e = threadIdx.x; e < n; e += blockDim.x) ss = fmaf(row[e], row[e], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    for (int e = threadIdx.x; e < n; e += blockDim.x)
        out[(size_t)blockIdx.x * n + e] = from_f32<TO>(row[e] * inv * (w ? w[e] : 1.0f));
}

template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* qproj, int q_stride, const float* proj, int stride,
                      const float* __restrict__ latent_weight, float eps,
                      const float* __restrict__ inv_freq, float mag, const int* __restrict__ positions,
                      const int* __restrict__ req_of_tok, const int* __restrict__ block_table, int bt_stride,
                      TC* __restrict__ pages, int num_pages, int page_size, int num_heads, int dk, int dr,
                      int rank, TQ* __restrict__ q_plain, TQ* __restrict__ q_full, int* __restrict__ status) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int qh = dk + dr, nq = num_heads * qh, row_len = rank + dr;
    const float* row = qproj + (size_t)t * q_stride;
    const int pos_i = positions[t];
    const float pos = (float)pos_i;
    for (int e = threadIdx.x; e < nq; e += blockDim.x) {
        const int j = e % qh, h = e / qh;
        if (j < dk) q_plain[((size_t)t * num_heads + h) * dk + j] = from_f32<TQ>(row[e]);
        else q_full[((size_t)t * num_heads + h) * row_len + rank + (j - dk)] =
                 from_f32<TQ>(mag * turned(row + h * qh + dk, j - dk, pos, inv_freq, 1.0f));
    }
    const int page = block_table[(size_t)req_of_tok[t] * bt_stride + pos_i / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
        return;
    }
    TC* dst = pages + ((size_t)page * page_size + pos_i % page_size) * row_len;
    const float* lat = proj + (size_t)t * stride;
    float ss = 0.0f;
    for (int e = threadIdx.x; e < rank; e += blockDim.x) ss = fmaf(lat[e], lat[e], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    for (int e = threadIdx.x; e < rank; e += blockDim.x)
        dst[e] = from_f32<TC>(lat[e] * inv * (latent_weight ? latent_weight[e] : 1.0f));
    for (int e = threadIdx.x; e < dr; e += blockDim.x)
        dst[rank + e] = from_f32<TC>(mag * turned(lat + rank, e, pos, inv_freq, 1.0f));
}

// out[t, h, n] = sum_k in[t, h, k] * w[h, k, n]; a block has 16 tokens of one head and 128 columns.
// Its eight warps take an eighth of k each, a lane four neighbouring columns (8 bytes of a weight row
// a load, eight loads in flight), so that a step of few tokens, whose grid is a block or a few per
// head, still has the weights of a head on their way at once; the tokens' inputs lie in shared
// memory with the tokens of one k side by side (read four at a time, the same address for the whole
// warp), and the warps' partial sums meet in shared memory in a fixed order.
constexpr int HP_TOKENS = 16;
constexpr int HP_WARPS = 8;

template <typename TW> __device__ __forceinline__ void load4(const TW* p, bool whole, int left, float (&w)[4]);
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, bool whole, int left, float (&w)[4]) {
    if (whole) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        w[0] = __bfloat162float(lo.x); w[1] = __bfloat162float(lo.y);
        w[2] = __bfloat162float(hi.x); w[3] = __bfloat162float(hi.y);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = i < left ? __bfloat162float(p[i]) : 0.0f;
    }
}
template <> __device__ __forceinline__ void load4<float>(const float* p, bool whole, int left, float (&w)[4]) {
    if (whole) {
        const float4 raw = *reinterpret_cast<const float4*>(p);
        w[0] = raw.x; w[1] = raw.y; w[2] = raw.z; w[3] = raw.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = i < left ? p[i] : 0.0f;
    }
}

template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(HP_WARPS * 32)
head_project_kernel(const TI* in, int in_stride_t, int in_stride_h, const TW* __restrict__ w, int n_in,
                    int n_out, TO* out, int out_stride_t, int out_stride_h, int num_tokens, int vec_ok) {
    extern __shared__ __align__(16) float xs[];      // [n_in][HP_TOKENS]; afterwards the warps' partial sums
    const int t0 = blockIdx.x * HP_TOKENS, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.z * 128 + lane * 4;      // this lane's first column
    const int nt = min(HP_TOKENS, num_tokens - t0);
    for (int e = threadIdx.x; e < HP_TOKENS * n_in; e += HP_WARPS * 32) {
        const int tt = e / n_in, k = e % n_in;
        xs[k * HP_TOKENS + tt] =
            tt < nt ? to_f32(in[(size_t)(t0 + tt) * in_stride_t + (size_t)h * in_stride_h + k]) : 0.0f;
    }
    __syncthreads();
    float acc[HP_TOKENS][4];
#pragma unroll
    for (int i = 0; i < HP_TOKENS; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    const int left = n_out - n0;                     // columns of this lane that exist
    if (left > 0) {
        const bool whole = vec_ok && left >= 4;
        const TW* wh = w + (size_t)h * n_in * n_out + n0;
        const int per = (n_in + HP_WARPS - 1) / HP_WARPS;
        const int k_end = min(n_in, (warp + 1) * per);
#pragma unroll 8
        for (int k = warp * per; k < k_end; ++k) {
            float wv[4];
            load4<TW>(wh + (size_t)k * n_out, whole, left, wv);
            const float4* x4 = reinterpret_cast<const float4*>(xs + k * HP_TOKENS);
#pragma unroll
            for (int i = 0; i < HP_TOKENS / 4; ++i) {
                const float4 x = x4[i];
                const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[4 * i + a][c] = fmaf(xv[a], wv[c], acc[4 * i + a][c]);
            }
        }
    }
    // the warps' sums meet in a fixed order (the upper half of the warps hands its sums to the lower
    // half, three times), so a row's bits are the same in every run
    float4* meet = reinterpret_cast<float4*>(xs);    // [warp][HP_TOKENS][32 lanes] of four columns
#pragma unroll
    for (int half = HP_WARPS / 2; half >= 1; half /= 2) {
        __syncthreads();                             // the inputs, or the round before, have been read
        if (warp >= half && warp < 2 * half) {
#pragma unroll
            for (int i = 0; i < HP_TOKENS; ++i)
                meet[((warp - half) * HP_TOKENS + i) * 32 + lane] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        }
        __syncthreads();
        if (warp < half) {
#pragma unroll
            for (int i = 0; i < HP_TOKENS; ++i) {
                const float4 o = meet[(warp * HP_TOKENS + i) * 32 + lane];
                acc[i][0] += o.x; acc[i][1] += o.y; acc[i][2] += o.z; acc[i][3] += o.w;
            }
        }
    }
    if (warp == 0 && left > 0) {
#pragma unroll
        for (int i = 0; i < HP_TOKENS; ++i) {
            if (i >= nt) break;
            TO* dst = out + (size_t)(t0 + i) * out_stride_t + (size_t)h * out_stride_h + n0;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (c < left) dst[c] = from_f32<TO>(acc[i][c]);
        }
    }
}

// The same product for many tokens, where the grid has blocks enough: four warps, a thread per column,
// all of k in one thread (no meeting of partial sums).
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(128)
head_project_rows_kernel(const TI* in, int in_stride_t, int in_stride_h, const TW* __restrict__ w, int n_in,
                         int n_out, TO* out, int out_stride_t, int out_stride_h, int num_tokens) {
    extern __shared__ __align__(16) float xs[];      // [n_in][HP_TOKENS]
    const int t0 = blockIdx.x * HP_TOKENS, h = blockIdx.y;
    const int n = blockIdx.z * 128 + threadIdx.x;
    const int nt = min(HP_TOKENS, num_tokens - t0);
    for (int e = threadIdx.x; e < HP_TOKENS * n_in; e += 128) {
        const int tt = e / n_in, k = e % n_in;
        xs[k * HP_TOKENS + tt] =
            tt < nt ? to_f32(in[(size_t)(t0 + tt) * in_stride_t + (size_t)h * in_stride_h + k]) : 0.0f;
    }
    __syncthreads();
    if (n >= n_out) return;
    float acc[HP_TOKENS];
#pragma unroll
    for (int i = 0; i < HP_TOKENS; ++i) acc[i] = 0.0f;
    const TW* wh = w + (size_t)h * n_in * n_out + n;
#pragma unroll 4
    for (int k = 0; k < n_in; ++k) {
        const float wv = to_f32(wh[(size_t)k * n_out]);
        const float4* x4 = reinterpret_cast<const float4*>(xs + k * HP_TOKENS);
#pragma unroll
        for (int i = 0; i < HP_TOKENS / 4; ++i) {
            const float4 x = x4[i];
            acc[4 * i] = fmaf(x.x, wv, acc[4 * i]);
            acc[4 * i + 1] = fmaf(x.y, wv, acc[4 * i + 1]);
            acc[4 * i + 2] = fmaf(x.z, wv, acc[4 * i + 2]);
            acc[4 * i + 3] = fmaf(x.w, wv, acc[4 * i + 3]);
        }
    }
#pragma unroll
    for (int i = 0; i < HP_TOKENS; ++i)
        if (i < nt) out[(size_t)(t0 + i) * out_stride_t + (size_t)h * out_stride_h + n] = from_f32<TO>(acc[i]);
}

struct AttnOptions {
    int window, chunk;            // 0: none
    float scale, softcap;         // softcap 0: none
    const float* head_scale;      // [heads] or null
    const float* sink;            // [heads] or null
    const float* gate;            // [T, gate_stride] float32 or null
    int gate_stride, gate_per_head, shared_rows;
};

template <typename TQ, typename TC, int PER_LANE>
__global__ void __launch_bounds__(WARPS * 32)
attention_options_kernel(const TQ* q, const int* __restrict__ rows, const int* __restrict__ positions,
                         const int* __restrict__ req_of_tok, const int* __restrict__ block_table,
                         int bt_stride, const TC* pages, int num_pages, int page_size, int num_heads,
                         int num_kv_heads, int dk, int dv, AttnOptions opt, TQ* __restrict__ out,
                         int* __restrict__ status) {
    __shared__ float so[WARPS][PER_LANE * 32];
    __shared__ float sm[WARPS], sl[WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, t = rows ? rows[blockIdx.x] : blockIdx.x;
    const int kvh = h / (num_heads / num_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)req_of_tok[t] * bt_stride;
    int lo = opt.window > 0 ? max(0, pos - opt.window + 1) : 0;
    if (opt.chunk > 0) lo = max(lo, pos / opt.chunk * opt.chunk);
    const size_t page_elems = (size_t)num_kv_heads * page_size * (opt.shared_rows ? dk : dk + dv);
    const size_t v_base = opt.shared_rows ? 0 : (size_t)num_kv_heads * page_size * dk;
    const int v_row = opt.shared_rows ? dk : dv;
    const float hs = opt.head_scale ? opt.scale * opt.head_scale[h] : opt.scale;

    float qv[PER_LANE], o[PER_LANE];
    const TQ* qh = q + ((size_t)t * num_heads + h) * dk;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < dk ? to_f32(qh[d]) : 0.0f;
        o[i] = 0.0f;
    }
    // the sink is one more logit without a value; the first warp starts from it
    float m = -INFINITY, l = 0.0f;
    if (opt.sink && warp == 0) { m = opt.sink[h]; l = 1.0f; }
    bool bad = false;
    for (int p = lo + warp; p <= pos; p += WARPS) {
        const int page = table[p / page_size];
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const TC* base = pages + (size_t)page * page_elems;
        const TC* kp = base + ((size_t)kvh * page_size + p % page_size) * dk;
        const TC* vp = base + v_base + ((size_t)kvh * page_size + p % page_size) * v_row;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < dk) s = fmaf(qv[i], to_f32(kp[d]), s);
        }
        s = warp_sum(s) * hs;
        if (opt.softcap > 0.0f) s = opt.softcap * tanhf(s / opt.softcap);
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);
        const float pr = expf(s - m_new);
        l = l * alpha + pr;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < dv) o[i] = fmaf(pr, to_f32(vp[d]), o[i] * alpha);
        }
        m = m_new;
    }
    if (bad && lane == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) so[warp][lane + 32 * i] = o[i];
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
    __syncthreads();
    if (warp == 0) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sm[w]);
        float ltot = 0.0f, wt[WARPS];
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            wt[w] = sl[w] > 0.0f ? expf(sm[w] - mm) : 0.0f;
            ltot += sl[w] * wt[w];
        }
        const float inv = 1.0f / ltot;
        TQ* oh = out + ((size_t)t * num_heads + h) * dv;
        const float* gt = opt.gate ? opt.gate + (size_t)t * opt.gate_stride : nullptr;
        const float head_gate = (gt && opt.gate_per_head) ? 1.0f / (1.0f + expf(-gt[h])) : 1.0f;
        for (int d = lane; d < dv; d += 32) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) acc = fmaf(so[w][d], wt[w], acc);
            acc *= inv * head_gate;
            if (gt && !opt.gate_per_head) acc *= 1.0f / (1.0f + expf(-gt[(size_t)h * dv + d]));
            oh[d] = from_f32<TQ>(acc);
        }
    }
}

// The same with a norm per head: every query head and every key head is divided by its own
// sqrt(mean(head^2) + eps) and multiplied by a weight of dk elements that all heads share.
// A warp takes a head; the values are copied by all.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
qk_headnorm_rope_store_kernel(const float* proj, int stride, const float* __restrict__ q_weight,
                              const float* __restrict__ k_weight, float eps,
                              const float* __restrict__ inv_freq, int rot,
                              const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                              const int* __restrict__ block_table, int bt_stride, TC* __restrict__ pages,
                              int num_pages, int page_size, int write_kv, int num_heads, int num_kv_heads,
                              int dk, int dv, TQ* __restrict__ q_out, int* __restrict__ status) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nq = num_heads * dk, nk = num_kv_heads * dk, nv = num_kv_heads * dv;
    const float* row = proj + (size_t)t * stride;
    const int pos_i = positions[t];
    const float pos = (float)pos_i;
    TC* base = nullptr;
    int slot = 0;
    if (write_kv) {
        const int page = block_table[(size_t)req_of_tok[t] * bt_stride + pos_i / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
            return;
        }
        slot = pos_i % page_size;
        base = pages + (size_t)page * num_kv_heads * page_size * (dk + dv);
    }
    const int units = num_heads + (write_kv ? num_kv_heads : 0);
    for (int u = warp; u < units; u += 8) {
        const bool is_q = u < num_heads;
        const int h = is_q ? u : u - num_heads;
        const float* head = row + (is_q ? 0 : nq) + (size_t)h * dk;
        const float* w = is_q ? q_weight : k_weight;
        float ss = 0.0f;
        for (int j = lane; j < dk; j += 32) ss = fmaf(head[j], head[j], ss);
        const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
        for (int j = lane; j < dk; j += 32) {
            float y;
            if (j < rot) {
                float s, c;
                sincosf(pos * inv_freq[j >> 1], &s, &c);
                const float a = head[j] * inv * (w ? w[j] : 1.0f);
                const float b = head[j ^ 1] * inv * (w ? w[j ^ 1] : 1.0f);
                y = (j & 1) ? a * c + b * s : a * c - b * s;
            } else {
                y = head[j] * inv * (w ? w[j] : 1.0f);
            }
            if (is_q) q_out[(size_t)t * nq + (size_t)h * dk + j] = from_f32<TQ>(y);
            else base[((size_t)h * page_size + slot) * dk + j] = from_f32<TC>(y);
        }
    }
    if (!write_kv) return;
    TC* vbase = base + (size_t)num_kv_heads * page_size * dk;
    const float* vrow = row + nq + nk;
    for (int e = threadIdx.x; e < nv; e += blockDim.x) {
        const int j = e % dv, g = e / dv;
        vbase[((size_t)g * page_size + slot) * dv + j] = from_f32<TC>(vrow[e]);
    }
}

}  // namespace

#define TI_DISPATCH_QC(qd, cd, CALL)                                               \
    if (qd == TI_F32 && cd == TI_F32) { CALL(float, float); }                      \
    else if (qd == TI_BF16 && cd == TI_BF16) { CALL(bf16, bf16); }                 \
    else if (qd == TI_F32 && cd == TI_BF16) { CALL(float, bf16); }                 \
    else return ti_fail("attention: dtype codes q=%d cache=%d are not supported", qd, cd);

extern "C" int ti_qk_rownorm_rope_store(const float* proj, int stride, const float* q_weight,
                                        const float* k_weight, float eps, const float* inv_freq, int rot,
                                        const int* positions, const int* req_of_tok, const int* block_table,
                                        int bt_stride, void* pages, int cache_dtype, int num_pages,
                                        int page_size, int write_kv, int num_tokens, int num_heads,
                                        int num_kv_heads, int dk, int dv, int per_head, void* q_out, int q_dtype,
                                        int* status, void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(rot >= 0 && rot <= dk && rot % 2 == 0, "qk_rownorm_rope_store: rotated width %d must be even "
               "and at most the head size %d", rot, dk);
    TI_REQUIRE(rot == 0 || inv_freq != nullptr, "qk_rownorm_rope_store: a rotation needs its frequencies");
    cudaStream_t s = (cudaStream_t)stream;
#define CALL(TQ, TC)                                                                              \
    (per_head ? qk_headnorm_rope_store_kernel<TQ, TC> : qk_rownorm_rope_store_kernel<TQ, TC>)<<<num_tokens, 256, 0, s>>>( \
        proj, stride, q_weight, k_weight, eps, inv_freq, rot, positions, req_of_tok, block_table,   \
        bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads, dk, dv,      \
        (TQ*)q_out, status)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
    return ti_check_launch("qk_rownorm_rope_store");
}

extern "C" int ti_slice_rmsnorm(const float* x, int stride, int num_rows, int n, const float* weight, float eps,
                                void* out, int out_dtype, void* stream) {
    if (num_rows == 0 || n == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == TI_BF16) slice_rmsnorm_kernel<bf16><<<num_rows, 256, 0, s>>>(x, stride, n, weight, eps, (bf16*)out);
    else if (out_dtype == TI_F32) slice_rmsnorm_kernel<float><<<num_rows, 256, 0, s>>>(x, stride, n, weight, eps, (float*)out);
    else return ti_fail("slice_rmsnorm: output dtype code %d", out_dtype);
    return ti_check_launch("slice_rmsnorm");
}

// `qproj` holds a token's query heads of (dk plain | dr rotated), `proj` its latent of `rank` and the key part of dr
extern "C" int ti_latent_prepare(const float* qproj, int q_stride, const float* proj, int stride,
                                 const float* latent_weight, float eps,
                                 const float* inv_freq, float mag, const int* positions, const int* req_of_tok,
                                 const int* block_table, int bt_stride, void* pages, int cache_dtype,
                                 int num_pages, int page_size, int num_tokens, int num_heads, int dk, int dr,
                                 int rank, void* q_plain, void* q_full, int q_dtype, int* status,
                                 void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(dr >= 0 && dr % 2 == 0, "latent_prepare: the rotated width %d must be even", dr);
    TI_REQUIRE(dr == 0 || inv_freq != nullptr, "latent_prepare: a rotation needs its frequencies");
    cudaStream_t s = (cudaStream_t)stream;
#define CALL(TQ, TC)                                                                              \
    latent_prepare_kernel<TQ, TC><<<num_tokens, 256, 0, s>>>(                                      \
        qproj, q_stride, proj, stride, latent_weight, eps, inv_freq, mag, positions, req_of_tok, block_table, bt_stride,  \
        (TC*)pages, num_pages, page_size, num_heads, dk, dr, rank, (TQ*)q_plain, (TQ*)q_full, status)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
    return ti_check_launch("latent_prepare");
}

extern "C" int ti_qkv_turn_store(const float* proj, int stride, const float* inv_freq, int rot, int halves, float mag,
                                 const float* v_inv_freq, int v_rot, int v_halves, const int* positions,
                                 const int* req_of_tok, const int* block_table, int bt_stride, void* pages,
                                 int cache_dtype, int num_pages, int page_size, int write_kv, int num_tokens,
                                 int num_heads, int num_kv_heads, int dk, int dv, void* q_out, int q_dtype,
                                 int* status, void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(rot >= 0 && rot <= dk && rot % 2 == 0, "qkv_turn_store: rotated width %d must be even and at most "
               "the head size %d", rot, dk);
    TI_REQUIRE(v_rot >= 0 && v_rot <= dv && v_rot % 2 == 0, "qkv_turn_store: rotated width %d of the values must be "
               "even and at most their head size %d", v_rot, dv);
    TI_REQUIRE((rot == 0 || inv_freq != nullptr) && (v_rot == 0 || v_inv_freq != nullptr),
               "qkv_turn_store: a rotation needs its frequencies");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t turn_smem = (size_t)(rot / 2 + v_rot / 2) * sizeof(float2);      // the token's cosines and sines
    TI_REQUIRE(turn_smem <= 48 * 1024, "qkv_turn_store: rotated widths %d and %d", rot, v_rot);
#define CALL(TQ, TC)                                                                              \
    qkv_turn_store_kernel<TQ, TC><<<num_tokens, 256, turn_smem, s>>>(                              \
        proj, stride, inv_freq, rot, halves, mag, v_inv_freq, v_rot, v_halves, positions, req_of_tok, \
        block_table, bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads, dk, dv, \
        (TQ*)q_out, status)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
    return ti_check_launch("qkv_turn_store");
}

extern "C" int ti_turn_rows(const void* x, int dtype, const int* positions, const float* inv_freq, int rot, int halves,
                            float sign, const float* gate, int gate_stride, int num_tokens, int num_heads, int n,
                            void* out, void* stream) {
    if (num_tokens == 0 || num_heads == 0) return 0;
    TI_REQUIRE(rot >= 0 && rot <= n && rot % 2 == 0, "turn_rows: rotated width %d must be even and at most %d", rot, n);
    TI_REQUIRE(rot == 0 || inv_freq != nullptr, "turn_rows: a rotation needs its frequencies");
    const size_t smem = (size_t)(rot / 2) * sizeof(float2);
    TI_REQUIRE(smem <= 48 * 1024, "turn_rows: a rotated width of %d", rot);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TI_BF16)
        turn_rows_kernel<bf16><<<num_tokens, 256, smem, s>>>((const bf16*)x, positions, inv_freq, rot, halves, sign, gate,
                                                            gate_stride, num_heads, n, (bf16*)out);
    else if (dtype == TI_F32)
        turn_rows_kernel<float><<<num_tokens, 256, smem, s>>>((const float*)x, positions, inv_freq, rot, halves, sign,
                                                             gate, gate_stride, num_heads, n, (float*)out);
    else return ti_fail("turn_rows: dtype code %d", dtype);
    return ti_check_launch("turn_rows");
}

extern "C" int ti_head_project(const void* in, int in_dtype, int in_stride_t, int in_stride_h, const void* w,
                               int w_dtype, int n_in, int n_out, void* out, int out_dtype, int out_stride_t,
                               int out_stride_h, int num_tokens, int num_heads, void* stream) {
    if (num_tokens == 0 || num_heads == 0) return 0;
    TI_REQUIRE(in_dtype == out_dtype, "head_project: input and output must have one dtype");
    size_t smem = (size_t)HP_TOKENS * n_in * sizeof(float);
    const size_t meet = (size_t)(HP_WARPS / 2) * HP_TOKENS * 128 * sizeof(float);     // where the warps' sums meet
    if (smem < meet) smem = meet;
    TI_REQUIRE(smem <= 48 * 1024, "head_project: %d inputs per head are more than the kernel stages", n_in);
    dim3 grid((num_tokens + HP_TOKENS - 1) / HP_TOKENS, num_heads, (n_out + 127) / 128);
    // four columns a load where every group of four starts on a multiple of the load's size
    const int vec_ok = n_out % 4 == 0 && (uintptr_t)w % 16 == 0;
    cudaStream_t s = (cudaStream_t)stream;
    // few blocks (a step of single tokens): the form whose warps split k, so that a head's weights are
    // on their way at once; many blocks: a thread per column with all of k.  (A row's bits can differ
    // between the two forms; within a form they depend on the row alone.)
    // Float32 rows always take the second form: their bits must not depend on the step around them.
    const bool few = in_dtype != TI_F32 && (long long)grid.x * grid.y * grid.z <= 512;
#define CALL(TI_, TW_)                                                                            \
    if (few)                                                                                      \
        head_project_kernel<TI_, TW_, TI_><<<grid, HP_WARPS * 32, smem, s>>>(                      \
            (const TI_*)in, in_stride_t, in_stride_h, (const TW_*)w, n_in, n_out, (TI_*)out,        \
            out_stride_t, out_stride_h, num_tokens, vec_ok);                                       \
    else                                                                                          \
        head_project_rows_kernel<TI_, TW_, TI_><<<grid, 128, smem, s>>>(                           \
            (const TI_*)in, in_stride_t, in_stride_h, (const TW_*)w, n_in, n_out, (TI_*)out,        \
            out_stride_t, out_stride_h, num_tokens)
    if (in_dtype == TI_F32 && w_dtype == TI_F32) { CALL(float, float); }
    else if (in_dtype == TI_F32 && w_dtype == TI_BF16) { CALL(float, bf16); }
    else if (in_dtype == TI_BF16 && w_dtype == TI_BF16) { CALL(bf16, bf16); }
    else return ti_fail("head_project: dtype codes in=%d w=%d are not supported", in_dtype, w_dtype);
#undef CALL
    return ti_check_launch("head_project");
}

// `rows` (may be null) lists the tokens to compute; without it all `num_rows` tokens are computed.
extern "C" int ti_attention_options(const void* q, int q_dtype, const int* rows, const int* positions,
                                    const int* req_of_tok, const int* block_table, int bt_stride,
                                    const void* pages, int cache_dtype, int num_pages, int page_size,
                                    int num_rows, int num_heads, int num_kv_heads, int dk, int dv,
                                    int shared_rows, int window, int chunk, float scale, float softcap,
                                    const float* head_scale, const float* sink, const float* gate,
                                    int gate_stride, int gate_per_head, void* out, int* status,
                                    void* stream) {
    if (num_rows == 0) return 0;
    const int widest = dk > dv ? dk : dv;
    TI_REQUIRE(dk >= 1 && dv >= 1 && widest <= 1024, "attention_options: head sizes %d and %d must be at "
               "most 1024", dk, dv);
    TI_REQUIRE(num_heads % num_kv_heads == 0, "attention_options: %d heads over %d kv heads", num_heads,
               num_kv_heads);
    TI_REQUIRE(!shared_rows || dv <= dk, "attention_options: a value of %d elements does not fit into a "
               "shared row of %d", dv, dk);
    TI_REQUIRE(window >= 0 && chunk >= 0 && softcap >= 0.0f, "attention_options: negative window, chunk or cap");
    AttnOptions opt = {window, chunk, scale, softcap, head_scale, sink, gate, gate_stride, gate_per_head,
                       shared_rows};
    dim3 grid(num_rows, num_heads);
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(TQ, TC, PL)                                                                         \
    attention_options_kernel<TQ, TC, PL><<<grid, WARPS * 32, 0, s>>>(                               \
        (const TQ*)q, rows, positions, req_of_tok, block_table, bt_stride, (const TC*)pages,          \
        num_pages, page_size, num_heads, num_kv_heads, dk, dv, opt, (TQ*)out, status)
#define CALL(TQ, TC)                                                                               \
    if (widest <= 128) LAUNCH(TQ, TC, 4); else if (widest <= 256) LAUNCH(TQ, TC, 8);                 \
    else if (widest <= 640) LAUNCH(TQ, TC, 20); else LAUNCH(TQ, TC, 32)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
#undef LAUNCH
    return ti_check_launch("attention_options");
}
