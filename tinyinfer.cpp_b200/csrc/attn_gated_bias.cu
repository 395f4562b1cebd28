// Attention with a learned bias per (head, distance), a window that keeps a request's first
// tokens, value heads of their own size and an output gate, on the CUDA cores.
//
//  * embed_sinusoid: x[t] = table[token[t]] * scale + s(pos[t]), where s(p)[2i] = sin(p f_i),
//    s(p)[2i + 1] = cos(p f_i) and f_i comes from the caller (float32); without frequencies the scaled
//    row alone.
//  * qkv_bias_norm_store: adds the projection's bias, brings every query and key head to unit
//    root mean square (times a weight, if one is given), writes keys and values once per kv head
//    into the token's page and the queries for the attention kernel.
//  * attention_bias_simple: one block per (token, query head).  Token i sees key j <= i when
//    i - j < window or j < keep_first; the score is (q . k) * scale + bias[head][min(i - j,
//    n_dist - 1)]; the output, normalised, is multiplied by sigmoid(gate) element by element.
//
// These are the true 32-bit kernels and the general path of the bfloat16 engine.  Cache layout:
// a page holds its keys [kv head][slot][dk] and behind them its values [kv head][slot][dv]; with
// dk = dv this is the layout of the other attention kernels.
#include "common.cuh"

namespace {

constexpr int MAX_HEAD_DIM = 256;
constexpr int WARPS = 4;

enum { TI_ERR_BAD_PAGE = 1 };

template <typename TW>
__global__ void __launch_bounds__(256)
embed_sinusoid_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                      const int* __restrict__ positions, const float* __restrict__ freq,
                      float scale, int width, float* __restrict__ out) {
    const int t = blockIdx.x;
    const TW* row = table + (size_t)ids[t] * width;
    const float pos = (float)positions[t];
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float wave = 0.0f;                      // no frequencies: the scaled row alone
        if (freq != nullptr) {
            const float angle = pos * freq[d >> 1];
            wave = (d & 1) ? cosf(angle) : sinf(angle);
        }
        out[(size_t)t * width + d] = to_f32(row[d]) * scale + wave;
    }
}

template <typename TQ, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
qkv_bias_norm_store_kernel(const float* qkv, int qkv_stride, const float* __restrict__ bias,
                           const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                           float eps, const int* __restrict__ positions,
                           const int* __restrict__ req_of_tok, const int* __restrict__ block_table,
                           int bt_stride, TC* __restrict__ pages, int num_pages, int page_size,
                           int write_kv, int num_heads, int num_kv_heads, int dk, int dv,
                           TQ* __restrict__ q_out, int* __restrict__ status) {
    __shared__ float vec[WARPS][MAX_HEAD_DIM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int item = blockIdx.y * WARPS + warp;
    const int items = num_heads + (write_kv ? 2 * num_kv_heads : 0);
    if (item >= items) return;
    const int nq = num_heads * dk, nk = num_kv_heads * dk;
    int kind, head;
    if (item < num_heads) { kind = 0; head = item; }
    else if (item < num_heads + num_kv_heads) { kind = 1; head = item - num_heads; }
    else { kind = 2; head = item - num_heads - num_kv_heads; }
    const int col = kind == 0 ? head * dk : kind == 1 ? nq + head * dk : nq + nk + head * dv;
    const float* src = qkv + (size_t)t * qkv_stride + col;
    const float* b = bias ? bias + col : nullptr;
    TC* dst = nullptr;
    if (kind != 0) {
        const int pos = positions[t];
        const int page = block_table[(size_t)req_of_tok[t] * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
            return;
        }
        const size_t page_elems = (size_t)num_kv_heads * page_size * (dk + dv);
        const int slot = pos % page_size;
        dst = pages + (size_t)page * page_elems +
              (kind == 1 ? ((size_t)head * page_size + slot) * dk
                         : (size_t)num_kv_heads * page_size * dk + ((size_t)head * page_size + slot) * dv);
    }
    if (kind == 2) {
        for (int d = lane; d < dv; d += 32) dst[d] = from_f32<TC>(src[d] + (b ? b[d] : 0.0f));
        return;
    }
    const float* w = kind == 0 ? q_weight : k_weight;
    float ss = 0.0f;
    for (int d = lane; d < dk; d += 32) {
        const float v = src[d] + (b ? b[d] : 0.0f);
        vec[warp][d] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dk + eps);
    __syncwarp();
    for (int d = lane; d < dk; d += 32) {
        float y = vec[warp][d] * inv;
        if (w) y *= w[d];
        if (kind == 0) q_out[(size_t)t * nq + head * dk + d] = from_f32<TQ>(y);
        else dst[d] = from_f32<TC>(y);
    }
}

template <typename TQ, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
attention_bias_simple_kernel(const TQ* __restrict__ q, const int* __restrict__ rows,
                             const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                             const int* __restrict__ block_table, int bt_stride,
                             const TC* __restrict__ pages, int num_pages, int page_size,
                             int num_heads, int num_kv_heads, int dk, int dv, int window,
                             int keep_first, float scale, const float* __restrict__ dist_bias,
                             int n_dist, const float* gate, int gate_stride,
                             TQ* __restrict__ out, int* __restrict__ status) {
    constexpr int PER_LANE = MAX_HEAD_DIM / 32;
    __shared__ float so[WARPS][MAX_HEAD_DIM];
    __shared__ float sm[WARPS], sl[WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, t = rows ? rows[blockIdx.x] : blockIdx.x;
    const int kvh = h / (num_heads / num_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)req_of_tok[t] * bt_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_kept = min(keep_first, lo);              // first tokens that lie behind the window
    const int n_keys = n_kept + (pos - lo + 1);
    const size_t page_elems = (size_t)num_kv_heads * page_size * (dk + dv);
    const size_t v_base = (size_t)num_kv_heads * page_size * dk;
    const float* bias_h = dist_bias ? dist_bias + (size_t)h * n_dist : nullptr;

    float qv[PER_LANE], o[PER_LANE];
    const TQ* qh = q + ((size_t)t * num_heads + h) * dk;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < dk ? to_f32(qh[d]) : 0.0f;
        o[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    bool bad = false;
    for (int idx = warp; idx < n_keys; idx += WARPS) {
        const int p = idx < n_kept ? idx : lo + (idx - n_kept);
        const int page = table[p / page_size];
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const TC* base = pages + (size_t)page * page_elems;
        const TC* kp = base + ((size_t)kvh * page_size + p % page_size) * dk;
        const TC* vp = base + v_base + ((size_t)kvh * page_size + p % page_size) * dv;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < dk) s = fmaf(qv[i], to_f32(kp[d]), s);
        }
        s = warp_sum(s) * scale;
        if (bias_h) s += bias_h[min(pos - p, n_dist - 1)];
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
    for (int i = 0; i < PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) so[warp][d] = o[i];
    }
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
        const float* gh = gate ? gate + (size_t)t * gate_stride + (size_t)h * dv : nullptr;
        for (int d = lane; d < dv; d += 32) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) acc = fmaf(so[w][d], wt[w], acc);
            acc *= inv;
            if (gh) acc *= 1.0f / (1.0f + expf(-gh[d]));
            oh[d] = from_f32<TQ>(acc);
        }
    }
}

}  // namespace

#define TI_DISPATCH_QC(qd, cd, CALL)                                               \
    if (qd == TI_F32 && cd == TI_F32) { CALL(float, float); }                      \
    else if (qd == TI_BF16 && cd == TI_BF16) { CALL(bf16, bf16); }                 \
    else if (qd == TI_F32 && cd == TI_BF16) { CALL(float, bf16); }                 \
    else return ti_fail("attention: dtype codes q=%d cache=%d are not supported", qd, cd);

extern "C" int ti_embed_sinusoid(const void* table, int table_dtype, const int* ids,
                                 const int* positions, const float* freq, float scale,
                                 int num_tokens, int width, float* out, void* stream) {
    if (num_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == TI_BF16)
        embed_sinusoid_kernel<bf16><<<num_tokens, 256, 0, s>>>((const bf16*)table, ids, positions, freq,
                                                               scale, width, out);
    else if (table_dtype == TI_F32)
        embed_sinusoid_kernel<float><<<num_tokens, 256, 0, s>>>((const float*)table, ids, positions,
                                                                freq, scale, width, out);
    else
        return ti_fail("embed_sinusoid: dtype code %d is not supported", table_dtype);
    return ti_check_launch("embed_sinusoid");
}

extern "C" int ti_qkv_bias_norm_store(const float* qkv, int qkv_stride, const float* bias,
                                      const float* q_weight, const float* k_weight, float eps,
                                      const int* positions, const int* req_of_tok,
                                      const int* block_table, int bt_stride, void* pages,
                                      int cache_dtype, int num_pages, int page_size, int write_kv,
                                      int num_tokens, int num_heads, int num_kv_heads, int dk, int dv,
                                      void* q_out, int q_dtype, int* status, void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(dk >= 1 && dk <= MAX_HEAD_DIM && dv >= 1 && dv <= MAX_HEAD_DIM,
               "qkv_bias_norm_store: head sizes %d and %d must be at most %d", dk, dv, MAX_HEAD_DIM);
    const int items = num_heads + (write_kv ? 2 * num_kv_heads : 0);
    dim3 grid(num_tokens, (items + WARPS - 1) / WARPS);
    cudaStream_t s = (cudaStream_t)stream;
#define CALL(TQ, TC)                                                                           \
    qkv_bias_norm_store_kernel<TQ, TC><<<grid, WARPS * 32, 0, s>>>(                             \
        qkv, qkv_stride, bias, q_weight, k_weight, eps, positions, req_of_tok, block_table,      \
        bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads, dk, dv,   \
        (TQ*)q_out, status)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
    return ti_check_launch("qkv_bias_norm_store");
}

// `rows` (may be null) lists the tokens to compute; without it all `num_rows` tokens are computed.
extern "C" int ti_attention_bias_simple(const void* q, int q_dtype, const int* rows,
                                        const int* positions, const int* req_of_tok,
                                        const int* block_table, int bt_stride, const void* pages,
                                        int cache_dtype, int num_pages, int page_size, int num_rows,
                                        int num_heads, int num_kv_heads, int dk, int dv, int window,
                                        int keep_first, float scale, const float* dist_bias,
                                        int n_dist, const float* gate, int gate_stride, void* out,
                                        int* status, void* stream) {
    if (num_rows == 0) return 0;
    TI_REQUIRE(dk >= 1 && dk <= MAX_HEAD_DIM && dv >= 1 && dv <= MAX_HEAD_DIM,
               "attention_bias: head sizes %d and %d must be at most %d", dk, dv, MAX_HEAD_DIM);
    TI_REQUIRE(num_heads % num_kv_heads == 0, "attention_bias: %d heads over %d kv heads",
               num_heads, num_kv_heads);
    TI_REQUIRE(dist_bias == nullptr || n_dist >= 1, "attention_bias: an empty bias table");
    TI_REQUIRE(keep_first >= 0 && window >= 0, "attention_bias: negative window or kept tokens");
    dim3 grid(num_rows, num_heads);
    cudaStream_t s = (cudaStream_t)stream;
#define CALL(TQ, TC)                                                                           \
    attention_bias_simple_kernel<TQ, TC><<<grid, WARPS * 32, 0, s>>>(                           \
        (const TQ*)q, rows, positions, req_of_tok, block_table, bt_stride, (const TC*)pages,     \
        num_pages, page_size, num_heads, num_kv_heads, dk, dv, window, keep_first, scale,         \
        dist_bias, n_dist, gate, gate_stride, (TQ*)out, status)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
    return ti_check_launch("attention_bias_simple");
}
