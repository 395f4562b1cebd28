// A routed feed-forward on the CUDA cores: the router's choice, and the experts' products for
// every operand type.
//
//  * router_topk: per token the `top` experts of largest logit (ties: the lower index) with the
//    sigmoid of their logits as weights (or, `softmax`, their share of the softmax over all
//    experts, not renormalised); one more column of the same product, if there is one,
//    becomes the sigmoid gate of a shared expert.
//  * router_choose: scores s = softmax over all outputs of the router; the choice looks at s + correction,
//    only inside the `keep` groups (of `groups` equal runs of neighbours) whose largest such value is
//    largest, and takes the `top` largest there (ties: the lower index); the weights are the chosen
//    outputs' s, as they are.
//  An index at or behind the number of stacked experts names an *identity expert*: it has no tensors, and
//  its output is the token's input times the weight.  The kernels below skip its products and add
//  `w h[t]` where the slots are summed.
//  * moe_gate_up_simple: y[t][s] = silu(w g) * (w u) with g = Wgate_e h_t, u = Wup_e h_t, e and w
//    the expert and weight of the token's slot s (an expert's gate and up rows are stacked in one
//    matrix, interleaved in strips of 8 or one after the other).  The weight stands for a scaling of the
//    expert's input: (Wgate (w h), Wup (w h)) = (w g, w u).  With another activation (glu.cuh) the
//    weight scales the expert's output: y = w act(g, u).
//  * moe_down_simple: out[t] += sum over the slots, in order, of Wdown_e y[t][s].
//  Both take a shared expert along when one is given: its gate/up products as one more pair per
//  token with weight 1, its down product added to the token's sum times the token's gate.
//  * scale_rows: y[t] *= f[t].
//
// These are the true 32-bit kernels and the general path of the bfloat16 engine; float32
// accumulation, k ascending inside a lane's share and a fixed butterfly across lanes, so a
// row's bits do not depend on what else is in the batch.
#include "common.cuh"
#include "glu.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_TOP = 32;

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// A lane's share of x . a and x . b over `n` elements.  bfloat16 operands whose rows are 16-byte
// aligned go eight elements a load (a warp then asks for 512 contiguous bytes of a weight row at
// once, instead of 64); everything else one element at a time.
template <typename TA, typename TW>
__device__ __forceinline__ void lane_dots(const TA* __restrict__ x, const TW* __restrict__ a, const TW* __restrict__ b,
                                          int n, int lane, float& ra, float& rb) {
    ra = rb = 0.0f;
    if constexpr (sizeof(TA) == 2 && sizeof(TW) == 2) {
        const bool vec = n % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)a % 16 == 0) &&
                         (b == nullptr || (uintptr_t)b % 16 == 0);
        if (vec) {
            for (int k = lane * 8; k < n; k += 256) {
                const uint4 xv = *reinterpret_cast<const uint4*>(x + k);
                const uint4 av = *reinterpret_cast<const uint4*>(a + k);
                const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
                const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&av);
                uint4 bv = make_uint4(0u, 0u, 0u, 0u);
                if (b != nullptr) bv = *reinterpret_cast<const uint4*>(b + k);
                const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 xf = __bfloat1622float2(xp[i]), af = __bfloat1622float2(ap[i]);
                    const float2 bf = __bfloat1622float2(bp[i]);
                    ra = fmaf(xf.x, af.x, ra); ra = fmaf(xf.y, af.y, ra);
                    rb = fmaf(xf.x, bf.x, rb); rb = fmaf(xf.y, bf.y, rb);
                }
            }
            return;
        }
    }
    for (int k = lane; k < n; k += 32) {
        const float xv = to_f32(x[k]);
        ra = fmaf(xv, to_f32(a[k]), ra);
        if (b != nullptr) rb = fmaf(xv, to_f32(b[k]), rb);
    }
}

__global__ void __launch_bounds__(WARPS * 32)
router_topk_kernel(const float* logits, int stride, int num_tokens, int experts, int top,
                   int shared_col, int* __restrict__ ids, float* __restrict__ weights,
                   float* __restrict__ shared_gate, int softmax) {
    __shared__ int chosen[WARPS][MAX_TOP];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * WARPS + warp;
    if (t >= num_tokens) return;
    const float* z = logits + (size_t)t * stride;
    // up to 256 experts: a lane's logits stay in registers, a chosen one is struck out there
    constexpr int HELD = 8;
    const bool held = experts <= 32 * HELD;
    float mine[HELD];
    bool gone[HELD];
#pragma unroll
    for (int i = 0; i < HELD; ++i) {
        const int e = lane + 32 * i;
        mine[i] = held && e < experts ? z[e] : 0.0f;
        gone[i] = !(held && e < experts);
    }
    float z_max = 0.0f, z_sum = 1.0f;                 // softmax over all experts: exp(z - max) / sum
    if (softmax) {
        float m = -INFINITY;
        for (int e = lane; e < experts; e += 32) m = fmaxf(m, z[e]);
        z_max = warp_max(m);
        float acc = 0.0f;
        for (int e = lane; e < experts; e += 32) acc += expf(z[e] - z_max);
        z_sum = warp_sum(acc);
    }
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int best_e = experts;                         // larger than every index: loses every tie
        if (held) {
#pragma unroll
            for (int i = 0; i < HELD; ++i) {
                const int e = lane + 32 * i;
                if (!gone[i] && (best_e == experts || mine[i] > best)) { best = mine[i]; best_e = e; }
            }
        } else {
            for (int e = lane; e < experts; e += 32) {
                bool taken = false;
                for (int c = 0; c < s; ++c) taken |= chosen[warp][c] == e;
                const float v = z[e];
                if (!taken && (v > best || (v == best && e < best_e) || best_e == experts)) { best = v; best_e = e; }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe < experts && (best_e == experts || ov > best || (ov == best && oe < best_e))) { best = ov; best_e = oe; }
        }
        best_e = __shfl_sync(0xffffffffu, best_e, 0);
        best = __shfl_sync(0xffffffffu, best, 0);
#pragma unroll
        for (int i = 0; i < HELD; ++i)
            if (lane + 32 * i == best_e) gone[i] = true;
        if (lane == 0) {
            chosen[warp][s] = best_e;
            ids[(size_t)t * top + s] = best_e;
            weights[(size_t)t * top + s] = softmax ? expf(best - z_max) / z_sum : sigmoidf_(best);
        }
        __syncwarp();
    }
    if (shared_col >= 0 && lane == 0) shared_gate[t] = sigmoidf_(z[shared_col]);
}

constexpr int MAX_ROUTED = 512;       // router outputs a warp keeps in shared memory
constexpr int MAX_GROUPS = 64;

__global__ void __launch_bounds__(WARPS * 32)
router_choose_kernel(const float* logits, int stride, int num_tokens, int total, int top,
                     const float* __restrict__ correction, int groups, int keep,
                     int* __restrict__ ids, float* __restrict__ weights) {
    __shared__ float choice[WARPS][MAX_ROUTED];
    __shared__ float group_best[WARPS][MAX_GROUPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * WARPS + warp;
    if (t >= num_tokens) return;
    const float* z = logits + (size_t)t * stride;
    float m = -INFINITY;
    for (int e = lane; e < total; e += 32) m = fmaxf(m, z[e]);
    const float z_max = warp_max(m);
    float acc = 0.0f;
    for (int e = lane; e < total; e += 32) acc += expf(z[e] - z_max);
    const float z_sum = warp_sum(acc);
    float* c = choice[warp];
    for (int e = lane; e < total; e += 32) c[e] = expf(z[e] - z_max) / z_sum + (correction ? correction[e] : 0.0f);
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = total / groups;
        float* gb = group_best[warp];
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, c[e]);
            gb[g] = b;
        }
        __syncwarp();
        // a group stays if fewer than `keep` groups come before it (a larger value, or the same and a lower index)
        for (int g = lane; g < groups; g += 32) {
            int before = 0;
            for (int o = 0; o < groups; ++o) before += gb[o] > gb[g] || (gb[o] == gb[g] && o < g);
            if (before >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
        }
        __syncwarp();
    }
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int best_e = total;                           // larger than every index: loses every tie
        for (int e = lane; e < total; e += 32) {
            const float v = c[e];
            if (v > best || (best_e == total && v > -INFINITY)) { best = v; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe < total && (best_e == total || ov > best || (ov == best && oe < best_e))) { best = ov; best_e = oe; }
        }
        best_e = __shfl_sync(0xffffffffu, best_e, 0);
        if (lane == 0) {
            // fewer outputs left than slots (a configuration the caller refuses): the slot gets weight 0
            ids[(size_t)t * top + s] = best_e < total ? best_e : 0;
            weights[(size_t)t * top + s] = best_e < total ? expf(z[best_e] - z_max) / z_sum : 0.0f;
            if (best_e < total) c[best_e] = -INFINITY;
        }
        __syncwarp();
    }
}

// one warp per output element f of one (token, slot)
template <typename TA, typename TW>
__global__ void __launch_bounds__(WARPS * 32)
moe_gate_up_simple_kernel(const TA* __restrict__ h, int h_stride, const TW* __restrict__ w_gate_up,
                          int interleaved, const int* __restrict__ ids,
                          const float* __restrict__ weights, int top, int width, int ff,
                          TA* __restrict__ y, int n_pairs, const TW* __restrict__ shared_gate_up,
                          int shared_interleaved, int shared_ff, TA* __restrict__ y_shared,
                          int act, float act_limit, float act_alpha, int experts) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int ts = blockIdx.x;                              // token * top + slot; behind the pairs: a token's shared expert
    const int f = blockIdx.y * WARPS + warp;
    const bool shared = ts >= n_pairs;
    if (shared) {
        ts -= n_pairs;                                // the token
        w_gate_up = shared_gate_up;
        interleaved = shared_interleaved;
        ff = shared_ff;
        y = y_shared;
    }
    if (f >= ff) return;
    const int e = shared ? 0 : ids[ts];
    if (e >= experts) return;                         // an identity expert: nothing to multiply
    const float w = shared ? 1.0f : weights[ts];
    const TA* x = h + (size_t)(shared ? ts : ts / top) * h_stride;
    // an expert's 2 ff rows: strips of 8 gate rows and their 8 up rows, or all gate rows and then all up rows
    const size_t gate_row = interleaved ? (size_t)(f >> 3) * 16 + (f & 7) : (size_t)f;
    const size_t up_row = interleaved ? gate_row + 8 : (size_t)ff + f;
    const TW* wg = w_gate_up + ((size_t)e * 2 * ff + gate_row) * width;
    const TW* wu = w_gate_up + ((size_t)e * 2 * ff + up_row) * width;
    float g, u;
    lane_dots(x, wg, wu, width, lane, g, u);
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) {
        // silu: the weight scales the expert's input; other activations: its output
        const float out = act == GLU_SILU ? (g * w) * sigmoidf_(g * w) * (u * w)
                                          : w * glu_activation(act, g, u, act_limit, act_alpha);
        y[(size_t)ts * ff + f] = from_f32<TA>(out);
    }
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(WARPS * 32)
moe_down_simple_kernel(const TA* __restrict__ y, const TW* __restrict__ w_down,
                       const int* __restrict__ ids, int top, int width, int ff,
                       float* __restrict__ out, int out_stride, const TA* __restrict__ y_shared,
                       const TW* __restrict__ w_shared_down, const float* __restrict__ shared_gate,
                       int shared_ff, int experts, const TA* __restrict__ h, int h_stride,
                       const float* __restrict__ weights) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int n = blockIdx.y * WARPS + warp;
    if (n >= width) return;
    float total = 0.0f;
    for (int s = 0; s < top; ++s) {
        const int e = ids[(size_t)t * top + s];
        if (e >= experts) {                           // an identity expert: the token's input times the weight
            total = fmaf(weights[(size_t)t * top + s], to_f32(h[(size_t)t * h_stride + n]), total);
            continue;
        }
        const TA* ys = y + ((size_t)t * top + s) * ff;
        const TW* wd = w_down + ((size_t)e * width + n) * ff;
        float acc, unused;
        lane_dots(ys, wd, (const TW*)nullptr, ff, lane, acc, unused);
        total += warp_sum(acc);
    }
    if (y_shared != nullptr) {                        // the shared expert's row, times the token's gate
        const TA* ys = y_shared + (size_t)t * shared_ff;
        const TW* wd = w_shared_down + (size_t)n * shared_ff;
        float acc, unused;
        lane_dots(ys, wd, (const TW*)nullptr, shared_ff, lane, acc, unused);
        total += warp_sum(acc) * shared_gate[t];
    }
    if (lane == 0) out[(size_t)t * out_stride + n] += total;
}

template <typename T>
__global__ void scale_rows_kernel(T* __restrict__ y, int stride, const float* __restrict__ f,
                                  int rows, int cols) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    const int r = (int)(i / cols), c = (int)(i % cols);
    T* p = y + (size_t)r * stride + c;
    *p = from_f32<T>(to_f32(*p) * f[r]);
}

}  // namespace

#define TI_DISPATCH_AW(ad, wd, CALL)                                               \
    if (ad == TI_F32 && wd == TI_F32) { CALL(float, float); }                      \
    else if (ad == TI_BF16 && wd == TI_BF16) { CALL(bf16, bf16); }                 \
    else if (ad == TI_F32 && wd == TI_BF16) { CALL(float, bf16); }                 \
    else if (ad == TI_BF16 && wd == TI_F32) { CALL(bf16, float); }                 \
    else return ti_fail("moe: dtype codes activations=%d weights=%d are not supported", ad, wd);

extern "C" int ti_router_topk(const float* logits, int stride, int num_tokens, int experts, int top,
                              int shared_col, int* ids, float* weights, float* shared_gate,
                              int softmax, void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(top >= 1 && top <= MAX_TOP && top <= experts,
               "router_topk: %d of %d experts (at most %d are chosen)", top, experts, MAX_TOP);
    router_topk_kernel<<<(num_tokens + WARPS - 1) / WARPS, WARPS * 32, 0, (cudaStream_t)stream>>>(
        logits, stride, num_tokens, experts, top, shared_col, ids, weights, shared_gate, softmax);
    return ti_check_launch("router_topk");
}

// `total` router outputs in `groups` equal groups of which `keep` may be chosen from (groups = 1: no groups);
// `correction` (may be null) is added to the scores for the choice alone.
extern "C" int ti_router_choose(const float* logits, int stride, int num_tokens, int total, int top,
                                const float* correction, int groups, int keep, int* ids, float* weights,
                                void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(total >= 1 && total <= MAX_ROUTED, "router_choose: %d router outputs (at most %d)", total, MAX_ROUTED);
    TI_REQUIRE(groups >= 1 && groups <= MAX_GROUPS && total % groups == 0 && keep >= 1 && keep <= groups,
               "router_choose: %d outputs in %d groups of which %d are kept", total, groups, keep);
    TI_REQUIRE(top >= 1 && top <= MAX_TOP && top <= total / groups * keep,
               "router_choose: %d of %d outputs cannot be chosen", top, total / groups * keep);
    router_choose_kernel<<<(num_tokens + WARPS - 1) / WARPS, WARPS * 32, 0, (cudaStream_t)stream>>>(
        logits, stride, num_tokens, total, top, correction, groups, keep, ids, weights);
    return ti_check_launch("router_choose");
}

extern "C" int ti_moe_gate_up_simple(const void* h, int act_dtype, int h_stride, const void* w_gate_up,
                                     int interleaved, int w_dtype, const int* ids,
                                     const float* weights, int num_tokens, int top, int width, int ff,
                                     void* y, const void* shared_gate_up, int shared_interleaved,
                                     int shared_ff, void* y_shared, int act, float act_limit,
                                     float act_alpha, int experts, void* stream) {
    if (num_tokens == 0) return 0;
    // with a shared expert (same weight dtype): one more "pair" per token behind the routed ones
    const bool shared = shared_gate_up != nullptr;
    const int most = shared && shared_ff > ff ? shared_ff : ff;
    dim3 grid(num_tokens * top + (shared ? num_tokens : 0), (most + WARPS - 1) / WARPS);
    cudaStream_t s = (cudaStream_t)stream;
#define CALL(TA, TW)                                                                         \
    moe_gate_up_simple_kernel<TA, TW><<<grid, WARPS * 32, 0, s>>>(                            \
        (const TA*)h, h_stride, (const TW*)w_gate_up, interleaved, ids, weights, top, width, ff, (TA*)y, \
        num_tokens * top, (const TW*)shared_gate_up, shared_interleaved, shared_ff, (TA*)y_shared, \
        act, act_limit, act_alpha, experts)
    TI_DISPATCH_AW(act_dtype, w_dtype, CALL)
#undef CALL
    return ti_check_launch("moe_gate_up_simple");
}

extern "C" int ti_moe_down_simple(const void* y, int act_dtype, const void* w_down, int w_dtype,
                                  const int* ids, int num_tokens, int top, int width, int ff,
                                  float* out, int out_stride, const void* y_shared,
                                  const void* w_shared_down, const float* shared_gate, int shared_ff,
                                  int experts, const void* h, int h_stride, const float* weights,
                                  void* stream) {
    if (num_tokens == 0) return 0;
    dim3 grid(num_tokens, (width + WARPS - 1) / WARPS);
    cudaStream_t s = (cudaStream_t)stream;
#define CALL(TA, TW)                                                                         \
    moe_down_simple_kernel<TA, TW><<<grid, WARPS * 32, 0, s>>>(                               \
        (const TA*)y, (const TW*)w_down, ids, top, width, ff, out, out_stride, (const TA*)y_shared, \
        (const TW*)w_shared_down, shared_gate, shared_ff, experts, (const TA*)h, h_stride, weights)
    TI_DISPATCH_AW(act_dtype, w_dtype, CALL)
#undef CALL
    return ti_check_launch("moe_down_simple");
}

extern "C" int ti_scale_rows(void* y, int dtype, int stride, const float* f, int rows, int cols,
                             void* stream) {
    if (rows == 0 || cols == 0) return 0;
    const size_t n = (size_t)rows * cols;
    const int blocks = (int)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TI_BF16) scale_rows_kernel<bf16><<<blocks, 256, 0, s>>>((bf16*)y, stride, f, rows, cols);
    else if (dtype == TI_F32) scale_rows_kernel<float><<<blocks, 256, 0, s>>>((float*)y, stride, f, rows, cols);
    else return ti_fail("scale_rows: dtype code %d is not supported", dtype);
    return ti_check_launch("scale_rows");
}
