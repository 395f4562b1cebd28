// Row-wise kernels around the recurrent mixers and the blocks that norm a sublayer's output.
//
//  * causal_conv_rows: a short causal convolution over time on every channel,
//        y[t, c] = sum_j w[c, j] x[t - taps + 1 + j, c]          (the last tap is the token's own),
//    where rows before a request's first token of this step come from the request's state (its last
//    taps - 1 inputs, zeros for a new request).  Options: add the input (x + conv(x)), silu on the
//    result.  With taps = 0 it converts the rows.  `conv_tail_store` then renews the state; it runs
//    as a launch of its own behind the convolution, so no block reads a state that another one
//    has already overwritten.  Where every request brings one token (`renew`), the one thread that
//    reads a request's kept rows of a channel moves them up itself.
//  * group_norm_rows: RMS norm in `groups` equal consecutive parts of a row, each divided by its
//    own sqrt(mean(x^2) + eps), the whole times a weight per element; stored (optionally for
//    gathered rows) or added to a float32 residual.
//  * depth_mix: hist[index] = x, and, with weights, x = sum_{j <= index} w[j] hist[j].
//  * add_scaled: dst += sa a + sb b.
//  * tanh_norm_rows: the norm without a mean or a variance, y = tanh(alpha x) w + b with one scalar alpha;
//    stored (optionally for gathered rows) or added to a float32 residual, like the norm in groups.
//    tanh_norm_pair: such a norm's rows are added to the residual and the sum passes a second such norm in the
//    same launch (the norm behind one sublayer and the norm in front of the next).
//  * cap_rows: x = cap tanh(x / cap), in place.
//  * add_row: x[t] += row for every row of x.
//  * glu_rows: y = act(gate, up) over a float32 product that holds gate and up columns (stacked, or
//    in strips of 8 and 8).  GLU_CLAMPED: g = min(g, limit), u = clamp(u, -limit, limit),
//    y = g sigmoid(alpha g) (u + 1).
//
// All arithmetic is float32.
#include <initializer_list>

#include "common.cuh"
#include "glu.cuh"

namespace {

constexpr int MAX_TAPS = 16;

template <typename TO>
__global__ void __launch_bounds__(256)
causal_conv_rows_kernel(const float* x, int x_stride, const float* __restrict__ w, int taps, int channels,
                        const int* __restrict__ req_of_tok, const int* __restrict__ cu_q,
                        const int* __restrict__ slots, const float* state, size_t state_stride,
                        size_t state_offset, int add_input, int silu, int renew, TO* __restrict__ out,
                        int out_stride) {
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const float cur = x[(size_t)t * x_stride + c];
    float y = (add_input || taps == 0) ? cur : 0.0f;
    if (taps > 0) {
        const int r = req_of_tok[t];
        const int i = t - cu_q[r];                        // index of the token in its request's portion
        const float* kept = taps > 1 ? state + (size_t)slots[r] * state_stride + state_offset : nullptr;   // [taps - 1][channels]
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;                // how many tokens before this one
            float v;
            if (back == 0) v = cur;
            else if (back <= i) v = x[(size_t)(t - back) * x_stride + c];
            else v = kept[(size_t)(taps - 1 - (back - i)) * channels + c];   // the state's last row is the newest
            acc = fmaf(w[(size_t)c * taps + j], v, acc);
        }
        y += acc;
        if (renew && taps > 1) {                           // one token a request: nobody else reads these rows
            float* rows = const_cast<float*>(kept);
            for (int j = 0; j + 2 < taps; ++j) rows[(size_t)j * channels + c] = rows[(size_t)(j + 1) * channels + c];
            rows[(size_t)(taps - 2) * channels + c] = cur;
        }
    }
    if (silu) y = y / (1.0f + expf(-y));
    out[(size_t)t * out_stride + c] = from_f32<TO>(y);
}

// state[slot] <- the last taps - 1 inputs of the request after this step: rows of this step, or,
// where the portion is shorter than that, the rows the state held moved up.
__global__ void __launch_bounds__(256)
conv_tail_store_kernel(const float* x, int x_stride, int taps, int channels, const int* __restrict__ cu_q,
                       const int* __restrict__ slots, float* state, size_t state_stride, size_t state_offset) {
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int t0 = cu_q[r], n = cu_q[r + 1] - t0, keep = taps - 1;
    if (n <= 0) return;
    float* kept = state + (size_t)slots[r] * state_stride + state_offset;
    float rows[MAX_TAPS];
    for (int j = 0; j < keep; ++j) {
        const int i = n - keep + j;                       // index in the portion of the row that lands in row j
        rows[j] = i >= 0 ? x[(size_t)(t0 + i) * x_stride + c] : kept[(size_t)(j + n) * channels + c];
    }
    for (int j = 0; j < keep; ++j) kept[(size_t)j * channels + c] = rows[j];
}

// `wpg` warps share a group (each a strided share of its elements; their sums of squares meet in
// shared memory in a fixed order); the block's warps take the groups `blockDim / 32 / wpg` at a time.
template <typename TO, bool ADD>
__global__ void __launch_bounds__(256)
group_norm_rows_kernel(const float* x, const float* __restrict__ w, const int* __restrict__ rows, int groups,
                       int n, float eps, TO* __restrict__ out, float* residual, int res_stride, int wpg) {
    __shared__ float part[8];
    const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * n;
    const int per = n / groups, at_once = nw / wpg, sub = warp % wpg;
    for (int g0 = 0; g0 < groups; g0 += at_once) {
        const int g = g0 + warp / wpg;
        const bool live = g < groups;
        const float* xg = xr + (size_t)g * per;
        float ss = 0.0f;
        if (live)
            for (int e = sub * 32 + lane; e < per; e += wpg * 32) ss = fmaf(xg[e], xg[e], ss);
        ss = warp_sum(ss);
        if (wpg > 1) {
            if (lane == 0) part[warp] = ss;
            __syncthreads();
            ss = 0.0f;
            for (int i = 0; i < wpg; ++i) ss += part[(warp / wpg) * wpg + i];
            __syncthreads();                              // before the next groups' sums land
        }
        if (!live) continue;
        const float inv = 1.0f / sqrtf(ss / (float)per + eps);
        for (int e = sub * 32 + lane; e < per; e += wpg * 32) {
            const float y = xg[e] * inv * w[g * per + e];
            if constexpr (ADD) residual[(size_t)r * res_stride + g * per + e] += y;
            else out[(size_t)r * n + g * per + e] = from_f32<TO>(y);
        }
    }
}

__global__ void __launch_bounds__(256)
depth_mix_kernel(float* x, float* hist, size_t layer_elems, int index, const float* __restrict__ w, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float cur = x[i];
    hist[(size_t)index * layer_elems + i] = cur;
    if (w == nullptr) return;
    float acc = 0.0f;
    for (int j = 0; j < index; ++j) acc = fmaf(w[j], hist[(size_t)j * layer_elems + i], acc);
    x[i] = fmaf(w[index], cur, acc);
}

__global__ void __launch_bounds__(256)
add_scaled_kernel(float* dst, int dst_stride, const float* a, float sa, const float* b, float sb, int rows,
                  int cols) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    const int r = (int)(i / cols), c = (int)(i % cols);
    float y = sa * a[i];
    if (b) y = fmaf(sb, b[i], y);
    dst[(size_t)r * dst_stride + c] += y;
}

template <typename TO>
__global__ void __launch_bounds__(256)
glu_rows_kernel(const float* gu, int inter, size_t total, int interleaved, int kind, float limit, float alpha,
                TO* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / inter;
    const int f = (int)(i % inter);
    const float* row = gu + t * 2 * (size_t)inter;
    const size_t gate_at = interleaved ? (size_t)(f >> 3) * 16 + (f & 7) : (size_t)f;
    const size_t up_at = interleaved ? gate_at + 8 : (size_t)inter + f;
    out[i] = from_f32<TO>(glu_activation(kind, row[gate_at], row[up_at], limit, alpha));
}

// y = tanh(alpha x) w + b over rows of n elements: element-wise; a block row of the grid per row of x, a thread
// four neighbouring columns (one 16-byte load) where the rows allow, else one
template <typename TO> __device__ __forceinline__ void store4(TO* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&lo);
    raw.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float tanh_norm_one(float x, float alpha, float w, float b) { return fmaf(tanhf(alpha * x), w, b); }

template <typename TO, bool ADD, int VEC>
__global__ void __launch_bounds__(256)
tanh_norm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, int n, float alpha,
                      const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out,
                      float* residual, int res_stride) {
    const size_t r = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (c >= n) return;
    const float* src = x + (rows ? (size_t)rows[r] : r) * n + c;
    if constexpr (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src), wv = *reinterpret_cast<const float4*>(w + c);
        const float4 bv = b ? *reinterpret_cast<const float4*>(b + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float y0 = tanh_norm_one(v.x, alpha, wv.x, bv.x), y1 = tanh_norm_one(v.y, alpha, wv.y, bv.y);
        const float y2 = tanh_norm_one(v.z, alpha, wv.z, bv.z), y3 = tanh_norm_one(v.w, alpha, wv.w, bv.w);
        if constexpr (ADD) {
            float4* dst = reinterpret_cast<float4*>(residual + r * res_stride + c);
            float4 o = *dst;
            o.x += y0; o.y += y1; o.z += y2; o.w += y3;
            *dst = o;
        } else {
            store4<TO>(out + r * n + c, y0, y1, y2, y3);
        }
    } else {
        const float y = tanh_norm_one(*src, alpha, w[c], b ? b[c] : 0.0f);
        if constexpr (ADD) residual[r * res_stride + c] += y;
        else out[r * n + c] = from_f32<TO>(y);
    }
}

// residual += tanh(a1 y) w1 + b1, then out = tanh(a2 residual) w2 + b2
template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
tanh_norm_pair_kernel(const float* __restrict__ y, int n, float a1, const float* __restrict__ w1,
                      const float* __restrict__ b1, float* residual, int res_stride, float a2,
                      const float* __restrict__ w2, const float* __restrict__ b2, TO* __restrict__ out) {
    const size_t r = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (c >= n) return;
    if constexpr (VEC == 4) {
        const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float4 v = *reinterpret_cast<const float4*>(y + r * n + c);
        const float4 w1v = *reinterpret_cast<const float4*>(w1 + c), w2v = *reinterpret_cast<const float4*>(w2 + c);
        const float4 b1v = b1 ? *reinterpret_cast<const float4*>(b1 + c) : zero;
        const float4 b2v = b2 ? *reinterpret_cast<const float4*>(b2 + c) : zero;
        float4* dst = reinterpret_cast<float4*>(residual + r * res_stride + c);
        float4 o = *dst;
        o.x += tanh_norm_one(v.x, a1, w1v.x, b1v.x); o.y += tanh_norm_one(v.y, a1, w1v.y, b1v.y);
        o.z += tanh_norm_one(v.z, a1, w1v.z, b1v.z); o.w += tanh_norm_one(v.w, a1, w1v.w, b1v.w);
        *dst = o;
        store4<TO>(out + r * n + c, tanh_norm_one(o.x, a2, w2v.x, b2v.x), tanh_norm_one(o.y, a2, w2v.y, b2v.y),
                   tanh_norm_one(o.z, a2, w2v.z, b2v.z), tanh_norm_one(o.w, a2, w2v.w, b2v.w));
    } else {
        float* x = residual + r * res_stride + c;
        const float sum = *x + tanh_norm_one(y[r * n + c], a1, w1[c], b1 ? b1[c] : 0.0f);
        *x = sum;
        out[r * n + c] = from_f32<TO>(tanh_norm_one(sum, a2, w2[c], b2 ? b2[c] : 0.0f));
    }
}

__global__ void cap_rows_kernel(float* __restrict__ x, size_t total, float cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] / cap);
}

__global__ void add_row_kernel(float* __restrict__ x, int stride, const float* __restrict__ row, int cols, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % cols);
    x[(i / cols) * stride + c] += row[c];
}

}  // namespace

extern "C" int ti_causal_conv_rows(const float* x, int x_stride, const float* w, int taps, int channels, int rows,
                                   const int* req_of_tok, const int* cu_q, const int* slots, const float* state,
                                   long long state_stride, long long state_offset, int add_input, int silu,
                                   int renew, void* out, int out_dtype, int out_stride, void* stream) {
    if (rows == 0 || channels == 0) return 0;
    TI_REQUIRE(taps >= 0 && taps <= MAX_TAPS, "causal_conv_rows: %d taps (at most %d)", taps, MAX_TAPS);
    TI_REQUIRE(taps <= 1 || state != nullptr, "causal_conv_rows: a convolution over time needs the state");
    dim3 grid(rows, (channels + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == TI_BF16)
        causal_conv_rows_kernel<bf16><<<grid, 256, 0, s>>>(x, x_stride, w, taps, channels, req_of_tok, cu_q, slots, state,
                                                           (size_t)state_stride, (size_t)state_offset, add_input, silu,
                                                           renew, (bf16*)out, out_stride);
    else if (out_dtype == TI_F32)
        causal_conv_rows_kernel<float><<<grid, 256, 0, s>>>(x, x_stride, w, taps, channels, req_of_tok, cu_q, slots, state,
                                                            (size_t)state_stride, (size_t)state_offset, add_input, silu,
                                                            renew, (float*)out, out_stride);
    else return ti_fail("causal_conv_rows: output dtype code %d", out_dtype);
    return ti_check_launch("causal_conv_rows");
}

extern "C" int ti_conv_tail_store(const float* x, int x_stride, int taps, int channels, const int* cu_q,
                                  const int* slots, int requests, float* state, long long state_stride,
                                  long long state_offset, void* stream) {
    if (requests == 0 || channels == 0 || taps <= 1) return 0;
    TI_REQUIRE(taps <= MAX_TAPS, "conv_tail_store: %d taps (at most %d)", taps, MAX_TAPS);
    dim3 grid((channels + 255) / 256, requests);
    conv_tail_store_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, x_stride, taps, channels, cu_q, slots, state,
                                                                    (size_t)state_stride, (size_t)state_offset);
    return ti_check_launch("conv_tail_store");
}

extern "C" int ti_group_norm_rows(const float* x, const float* w, const int* rows, int num_rows, int n, int groups,
                                  float eps, void* out, int out_dtype, float* residual, int res_stride, void* stream) {
    if (num_rows == 0) return 0;
    TI_REQUIRE(groups >= 1 && n % groups == 0, "group_norm_rows: %d elements do not fall into %d equal groups", n, groups);
    cudaStream_t s = (cudaStream_t)stream;
    const int wpg = groups >= 8 ? 1 : 8 / groups;         // warps a group: 8, 4, 2, 2, 1, 1, 1, 1 for 1 to 8 groups
    const int threads = (groups >= 8 ? 8 : groups) * wpg * 32;
    if (residual != nullptr) {
        TI_REQUIRE(rows == nullptr, "group_norm_rows: rows are not gathered when adding to a residual");
        group_norm_rows_kernel<float, true><<<num_rows, threads, 0, s>>>(x, w, rows, groups, n, eps, nullptr, residual,
                                                                        res_stride, wpg);
    } else if (out_dtype == TI_BF16) {
        group_norm_rows_kernel<bf16, false><<<num_rows, threads, 0, s>>>(x, w, rows, groups, n, eps, (bf16*)out, nullptr, 0, wpg);
    } else if (out_dtype == TI_F32) {
        group_norm_rows_kernel<float, false><<<num_rows, threads, 0, s>>>(x, w, rows, groups, n, eps, (float*)out, nullptr, 0, wpg);
    } else {
        return ti_fail("group_norm_rows: output dtype code %d", out_dtype);
    }
    return ti_check_launch("group_norm_rows");
}

extern "C" int ti_depth_mix(float* x, float* hist, long long layer_elems, int index, const float* w, void* stream) {
    if (layer_elems == 0) return 0;
    const int blocks = (int)((layer_elems + 255) / 256);
    depth_mix_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, hist, (size_t)layer_elems, index, w, (size_t)layer_elems);
    return ti_check_launch("depth_mix");
}

extern "C" int ti_add_scaled(float* dst, int dst_stride, const float* a, float sa, const float* b, float sb, int rows,
                             int cols, void* stream) {
    if (rows == 0 || cols == 0) return 0;
    const size_t n = (size_t)rows * cols;
    add_scaled_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dst, dst_stride, a, sa, b, sb, rows, cols);
    return ti_check_launch("add_scaled");
}

extern "C" int ti_glu_rows(const float* gu, int num_tokens, int inter, int interleaved, int kind, float limit,
                           float alpha, void* out, int out_dtype, void* stream) {
    TI_REQUIRE(!interleaved || inter % 8 == 0, "glu_rows: the strip layout needs a multiple of 8 columns, got %d", inter);
    TI_REQUIRE(kind == GLU_SILU || kind == GLU_CLAMPED, "glu_rows: activation kind %d", kind);
    const size_t total = (size_t)num_tokens * inter;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == TI_BF16)
        glu_rows_kernel<bf16><<<blocks, 256, 0, s>>>(gu, inter, total, interleaved, kind, limit, alpha, (bf16*)out);
    else if (out_dtype == TI_F32)
        glu_rows_kernel<float><<<blocks, 256, 0, s>>>(gu, inter, total, interleaved, kind, limit, alpha, (float*)out);
    else return ti_fail("glu_rows: output dtype code %d", out_dtype);
    return ti_check_launch("glu_rows");
}

static bool rows_of_four(int n, int res_stride, std::initializer_list<const void*> ptrs) {
    if (n % 4 || res_stride % 4) return false;
    for (const void* p : ptrs)
        if ((uintptr_t)p % 16) return false;
    return true;
}

extern "C" int ti_tanh_norm_rows(const float* x, const int* rows, int num_rows, int n, float alpha, const float* w,
                                 const float* b, void* out, int out_dtype, float* residual, int res_stride, void* stream) {
    if (num_rows == 0 || n == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool four = rows_of_four(n, residual ? res_stride : 0, {x, w, b, out, residual});
    const dim3 grid(num_rows, (n + (four ? 1023 : 255)) / (four ? 1024 : 256));
    TI_REQUIRE(grid.y <= 65535, "tanh_norm_rows: rows of %d elements", n);
#define CALL(TO, ADD, VEC)                                                                            \
    tanh_norm_rows_kernel<TO, ADD, VEC><<<grid, 256, 0, s>>>(x, rows, n, alpha, w, b, (TO*)(ADD ? nullptr : out), \
                                                             residual, res_stride)
    if (residual != nullptr) {
        TI_REQUIRE(rows == nullptr, "tanh_norm_rows: rows are not gathered when adding to a residual");
        if (four) CALL(float, true, 4); else CALL(float, true, 1);
    } else if (out_dtype == TI_BF16) {
        if (four) CALL(bf16, false, 4); else CALL(bf16, false, 1);
    } else if (out_dtype == TI_F32) {
        if (four) CALL(float, false, 4); else CALL(float, false, 1);
    } else {
        return ti_fail("tanh_norm_rows: output dtype code %d", out_dtype);
    }
#undef CALL
    return ti_check_launch("tanh_norm_rows");
}

extern "C" int ti_cap_rows(float* x, long long total, float cap, void* stream) {
    if (total == 0) return 0;
    TI_REQUIRE(cap > 0.0f, "cap_rows: the cap must be positive");
    cap_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, (size_t)total, cap);
    return ti_check_launch("cap_rows");
}

extern "C" int ti_add_row(float* x, int stride, const float* row, int rows, int cols, void* stream) {
    const size_t total = (size_t)rows * cols;
    if (total == 0) return 0;
    add_row_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, stride, row, cols, total);
    return ti_check_launch("add_row");
}

extern "C" int ti_tanh_norm_pair(const float* y, int num_rows, int n, float a1, const float* w1, const float* b1,
                                 float* residual, int res_stride, float a2, const float* w2, const float* b2, void* out,
                                 int out_dtype, void* stream) {
    if (num_rows == 0 || n == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool four = rows_of_four(n, res_stride, {y, w1, b1, w2, b2, out, residual});
    const dim3 grid(num_rows, (n + (four ? 1023 : 255)) / (four ? 1024 : 256));
    TI_REQUIRE(grid.y <= 65535, "tanh_norm_pair: rows of %d elements", n);
#define CALL(TO, VEC) \
    tanh_norm_pair_kernel<TO, VEC><<<grid, 256, 0, s>>>(y, n, a1, w1, b1, residual, res_stride, a2, w2, b2, (TO*)out)
    if (out_dtype == TI_BF16) { if (four) CALL(bf16, 4); else CALL(bf16, 1); }
    else if (out_dtype == TI_F32) { if (four) CALL(float, 4); else CALL(float, 1); }
    else return ti_fail("tanh_norm_pair: output dtype code %d", out_dtype);
#undef CALL
    return ti_check_launch("tanh_norm_pair");
}
