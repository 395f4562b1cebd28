// The experts' products of a routed feed-forward on the tensor cores (bfloat16, mma.sync), for
// steps of many tokens.
//
//  1. moe_sort (one block): counts the (token, slot) pairs of every expert, lays the experts'
//     pairs out one after the other (`sorted_slot[pos]` = token * top + slot) and lists the
//     tiles of 64 rows, each inside one expert: {expert, first row, rows}.
//  2. moe_grouped<GATED>: a block takes one tile of rows and 64 output columns of its expert:
//     rows of h gathered by token, the expert's gate and up rows, float32 accumulation, and
//     y = silu(w g) * (w u) in the epilogue (w: the pair's weight), stored in sorted order; with
//     another activation (glu.cuh) the weight scales the output instead: y = w act(g, u).
//  3. moe_grouped<!GATED>: the same walk over y and the expert's down rows, 128 output columns a
//     block; the float32 result goes to the pair's own row of a scratch.
//  4. moe_combine: residual[t] += the rows of t's pairs, in slot order.
//
// Steps of very many tokens take the tcgen05 product of gemm_tcgen05.cu in its grouped form
// instead of 2 and 3; this file then brings what surrounds it: moe_sort_padded (every expert's
// pairs padded to whole tiles of 128 rows), moe_gather_scaled (the rows of h times their weights,
// in that order) and moe_combine_rows.
//
// No atomics touch a result, so a row's bits depend on its own operands only.  K is walked in
// steps of 32 through a three-stage cp.async ring; warps are arranged 2 x 2 over a 64 x 128
// tile of products (GATED: 64 gate and 64 up columns, interleaved in runs of 32 so that a warp
// holds both values of its 32 outputs).
#include "common.cuh"
#include "glu.cuh"

namespace {

constexpr int BM = 64, BNW = 128, BK = 32, STAGES = 3, THREADS = 128;
constexpr int ROW_BYTES = BK * 2 + 16;                 // padded: ldmatrix rows fall in distinct banks
constexpr int STAGE_BYTES = (BM + BNW) * ROW_BYTES;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The pairs of every expert counted in shared memory by one block; a thread has SORT_UNROLL loads
// of ids in flight at once (with one at a time the block waited a round trip per 1,024 pairs).
constexpr int SORT_UNROLL = 8;
__device__ __forceinline__ void count_pairs(const int* __restrict__ ids, int n_pairs, int experts, int* counts) {
    for (int base = threadIdx.x; base < n_pairs; base += blockDim.x * SORT_UNROLL) {
        int e[SORT_UNROLL];
#pragma unroll
        for (int u = 0; u < SORT_UNROLL; ++u) {
            const int i = base + u * blockDim.x;
            e[u] = i < n_pairs ? __ldg(ids + i) : -1;
        }
#pragma unroll
        for (int u = 0; u < SORT_UNROLL; ++u)
            if (e[u] >= 0 && e[u] < experts) atomicAdd(&counts[e[u]], 1);
    }
}

// meta: [0] = number of tiles.  tiles: [max_tiles][3] = {expert, first sorted row, rows}.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int experts, int* __restrict__ sorted_slot,
                int* __restrict__ tiles, int* __restrict__ meta) {
    extern __shared__ int sh[];                         // counts[experts], offsets[experts]
    int* counts = sh;
    int* offsets = sh + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    count_pairs(ids, n_pairs, experts, counts);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = at;
            for (int r = 0; r < counts[e]; r += BM) {
                tiles[nt * 3] = e;
                tiles[nt * 3 + 1] = at + r;
                tiles[nt * 3 + 2] = min(BM, counts[e] - r);
                ++nt;
            }
            at += counts[e];
            counts[e] = 0;                              // becomes the expert's cursor
        }
        meta[0] = nt;
    }
    __syncthreads();
    // the order of an expert's pairs among themselves is left to the atomics: every row of a
    // product is computed from its own operands alone, so no result depends on it
    for (int base = threadIdx.x; base < n_pairs; base += blockDim.x * SORT_UNROLL) {
        int e[SORT_UNROLL];
#pragma unroll
        for (int u = 0; u < SORT_UNROLL; ++u) {
            const int i = base + u * blockDim.x;
            e[u] = i < n_pairs ? __ldg(ids + i) : -1;
        }
#pragma unroll
        for (int u = 0; u < SORT_UNROLL; ++u)
            if (e[u] >= 0 && e[u] < experts)
                sorted_slot[offsets[e[u]] + atomicAdd(&counts[e[u]], 1)] = base + u * blockDim.x;
    }
}

template <bool GATED>
__global__ void __launch_bounds__(THREADS)
moe_grouped_kernel(const bf16* a, int lda, const int* __restrict__ sorted_slot,
                   const int* __restrict__ tiles, const int* __restrict__ meta, int top,
                   const bf16* __restrict__ w0, int interleaved, int n, int k,
                   const float* __restrict__ weights, bf16* __restrict__ y_sorted,
                   float* __restrict__ out_rows, int act, float act_limit, float act_alpha) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int row_src[BM];                         // the row of `a` behind each row of the tile
    const int tile = blockIdx.y;
    if (tile >= meta[0]) return;
    const int expert = tiles[tile * 3], row0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    constexpr int BN_OUT = GATED ? BNW / 2 : BNW;       // output columns of a block
    const int n0 = blockIdx.x * BN_OUT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp >> 1, wn = warp & 1;
    const int g = lane >> 2, tq = lane & 3;

    if (threadIdx.x < BM) {
        const int r = threadIdx.x;
        int src = -1;
        if (r < rows) src = GATED ? sorted_slot[row0 + r] / top : row0 + r;
        row_src[r] = src;
    }
    __syncthreads();
    // GATED: the expert's 2n rows (strips of 8 gate rows and their 8 up rows, or gate rows then up rows)
    const bf16* wg = w0 + (size_t)expert * (GATED ? 2 : 1) * n * k;

    // the weight row behind row r of the stage's B part
    auto b_row = [&](int r) -> const bf16* {
        if (GATED) {
            const int half = r >> 6, in = r & 63;
            const int col = n0 + half * 32 + (in & 31);
            if (col >= n) return nullptr;
            const size_t gate_row = interleaved ? (size_t)(col >> 3) * 16 + (col & 7) : (size_t)col;
            const size_t row = in < 32 ? gate_row : (interleaved ? gate_row + 8 : (size_t)n + col);
            return wg + row * k;
        }
        const int col = n0 + r;
        return col < n ? wg + (size_t)col * k : nullptr;
    };
    auto issue = [&](int kb, int stage) {
        unsigned char* as = smem + (size_t)stage * STAGE_BYTES;
        unsigned char* bs = as + BM * ROW_BYTES;
        const int k0 = kb * BK;
        for (int c = threadIdx.x; c < BM * 4; c += THREADS) {
            const int r = c >> 2, ch = c & 3;
            const int src = row_src[r];
            cp_async16(as + r * ROW_BYTES + ch * 16, src >= 0 ? a + (size_t)src * lda + k0 + ch * 8 : a, src >= 0);
        }
        for (int c = threadIdx.x; c < BNW * 4; c += THREADS) {
            const int r = c >> 2, ch = c & 3;
            const bf16* src = b_row(r);
            cp_async16(bs + r * ROW_BYTES + ch * 16, src ? src + k0 + ch * 8 : w0, src != nullptr);
        }
    };

    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

    const int kbs = k / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < kbs) issue(s, s);
        cp_async_commit();
    }
    for (int kb = 0; kb < kbs; ++kb) {
        if (kb + STAGES - 1 < kbs) issue(kb + STAGES - 1, (kb + STAGES - 1) % STAGES);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        const unsigned char* as = smem + (size_t)(kb % STAGES) * STAGE_BYTES;
        const unsigned char* bs = as + BM * ROW_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            unsigned af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(af[i], as + (wm * 32 + i * 16 + (lane & 15)) * ROW_BYTES + (kk * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                unsigned b[4];
                const int col = wn * 64 + jp * 16 + (lane >> 4) * 8 + (lane & 7);
                const int kd = kk * 16 + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(b, bs + col * ROW_BYTES + kd * 2);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma_bf16(acc[i][2 * jp], af[i], b[0], b[1]);
                    mma_bf16(acc[i][2 * jp + 1], af[i], b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * 32 + i * 16 + g + 8 * half;
            if (r >= rows) continue;
            if (GATED) {
                const float w = weights[sorted_slot[row0 + r]];
                bf16* dst = y_sorted + (size_t)(row0 + r) * n;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int col = n0 + wn * 32 + j * 8 + tq * 2;
                    if (col >= n) continue;
                    const float g0 = acc[i][j][2 * half] * w, g1 = acc[i][j][2 * half + 1] * w;
                    const float u0 = acc[i][j + 4][2 * half] * w, u1 = acc[i][j + 4][2 * half + 1] * w;
                    float y0, y1;
                    if (act == GLU_SILU) {               // the weight scales the expert's input
                        y0 = g0 / (1.0f + __expf(-g0)) * u0;
                        y1 = g1 / (1.0f + __expf(-g1)) * u1;
                    } else {                             // the weight scales the expert's output
                        y0 = w * glu_activation(act, acc[i][j][2 * half], acc[i][j + 4][2 * half], act_limit, act_alpha);
                        y1 = w * glu_activation(act, acc[i][j][2 * half + 1], acc[i][j + 4][2 * half + 1], act_limit, act_alpha);
                    }
                    *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(y0, y1);
                }
            } else {
                float* dst = out_rows + (size_t)sorted_slot[row0 + r] * n;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int col = n0 + wn * 64 + j * 8 + tq * 2;
                    if (col >= n) continue;
                    *reinterpret_cast<float2*>(dst + col) = make_float2(acc[i][j][2 * half], acc[i][j][2 * half + 1]);
                }
            }
        }
    }
}

// A slot whose index is not below `experts` names an identity expert: its row is the token's input times
// the slot's weight (`ids` null: there are none).
__global__ void moe_combine_kernel(const float* __restrict__ rows, int top, int width, int num_tokens,
                                   float* __restrict__ residual, int res_stride, const int* __restrict__ ids,
                                   int experts, const float* __restrict__ id_weights, const bf16* __restrict__ h,
                                   int h_stride) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)num_tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    float total = 0.0f;
    for (int s = 0; s < top; ++s) {
        if (ids != nullptr && ids[t * top + s] >= experts)
            total = fmaf(id_weights[t * top + s], __bfloat162float(h[(size_t)t * h_stride + c]), total);
        else
            total += rows[((size_t)t * top + s) * width + c];
    }
    residual[(size_t)t * res_stride + c] += total;
}

// For the grouped tcgen05 product: every expert's pairs padded to whole tiles of 128 rows.
// row_pair[row] = pair behind a row (-1: padding), pos_of_pair[pair] = its row,
// group_of_tile[i] = expert of row tile i, tiles_m[0] = number of row tiles.
__global__ void __launch_bounds__(1024)
moe_sort_padded_kernel(const int* __restrict__ ids, int n_pairs, int experts, int max_rows,
                       int* __restrict__ row_pair, int* __restrict__ pos_of_pair,
                       int* __restrict__ group_of_tile, int* __restrict__ tiles_m) {
    extern __shared__ int sh[];
    int* counts = sh;
    int* offsets = sh + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x) row_pair[r] = -1;
    __syncthreads();
    count_pairs(ids, n_pairs, experts, counts);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = at;
            const int t = (counts[e] + 127) / 128;
            for (int r = 0; r < t; ++r) group_of_tile[nt++] = e;
            at += t * 128;
            counts[e] = 0;
        }
        tiles_m[0] = nt;
    }
    __syncthreads();
    for (int base = threadIdx.x; base < n_pairs; base += blockDim.x * SORT_UNROLL) {
        int e[SORT_UNROLL];
#pragma unroll
        for (int u = 0; u < SORT_UNROLL; ++u) {
            const int i = base + u * blockDim.x;
            e[u] = i < n_pairs ? __ldg(ids + i) : -1;
        }
#pragma unroll
        for (int u = 0; u < SORT_UNROLL; ++u) {
            if (e[u] < 0 || e[u] >= experts) continue;
            const int i = base + u * blockDim.x;
            const int pos = offsets[e[u]] + atomicAdd(&counts[e[u]], 1);
            row_pair[pos] = i;
            pos_of_pair[i] = pos;
        }
    }
}

// a[row] = bfloat16(w * h[token]) for the pair behind the row, zeros for padding; 8 elements a thread
__global__ void moe_gather_scaled_kernel(const bf16* __restrict__ h, int h_stride, const int* __restrict__ row_pair,
                                         const int* __restrict__ tiles_m, const float* __restrict__ weights,
                                         int top, int width, bf16* __restrict__ a) {
    const int row = blockIdx.x;
    if (row >= tiles_m[0] * 128) return;
    const int pair = row_pair[row];
    const float w = pair >= 0 ? (weights != nullptr ? weights[pair] : 1.0f) : 0.0f;     // no weights: the rows as they are
    const bf16* src = h + (size_t)(pair >= 0 ? pair / top : 0) * h_stride;
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (pair >= 0) {
            v = *reinterpret_cast<const uint4*>(src + c);
            __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                p[i] = __floats2bfloat162_rn(f.x * w, f.y * w);
            }
        }
        *reinterpret_cast<uint4*>(a + (size_t)row * width + c) = v;
    }
}

__global__ void moe_combine_rows_kernel(const float* __restrict__ rows, const int* __restrict__ pos_of_pair, int top,
                                        int width, int num_tokens, float* __restrict__ residual, int res_stride,
                                        const float* __restrict__ weights, const int* __restrict__ ids, int experts,
                                        const float* __restrict__ id_weights, const bf16* __restrict__ h, int h_stride) {
    const int quads = width >> 2;                      // width is a multiple of 8 on this path
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)num_tokens * quads) return;
    const int t = (int)(i / quads), c = (int)(i % quads) * 4;
    float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < top; ++s) {
        if (ids != nullptr && ids[t * top + s] >= experts) {      // an identity expert: the input times the weight
            const float w = id_weights[t * top + s];
            const bf16* x = h + (size_t)t * h_stride + c;
            total.x = fmaf(w, __bfloat162float(x[0]), total.x); total.y = fmaf(w, __bfloat162float(x[1]), total.y);
            total.z = fmaf(w, __bfloat162float(x[2]), total.z); total.w = fmaf(w, __bfloat162float(x[3]), total.w);
            continue;
        }
        const float4 v = *reinterpret_cast<const float4*>(rows + (size_t)pos_of_pair[t * top + s] * width + c);
        const float w = weights != nullptr ? weights[t * top + s] : 1.0f;            // a pair's weight on its expert's output
        total.x = fmaf(w, v.x, total.x); total.y = fmaf(w, v.y, total.y);
        total.z = fmaf(w, v.z, total.z); total.w = fmaf(w, v.w, total.w);
    }
    float* dst = residual + (size_t)t * res_stride + c;
    dst[0] += total.x; dst[1] += total.y; dst[2] += total.z; dst[3] += total.w;
}

}  // namespace

// The pieces around the grouped tcgen05 product.  max_rows = (pairs / 128 + experts) * 128.
extern "C" int ti_moe_sort_padded(const int* ids, int num_pairs, int experts, int max_rows, int* row_pair,
                                  int* pos_of_pair, int* group_of_tile, int* tiles_m, void* stream) {
    TI_REQUIRE(experts >= 1 && experts <= 4096, "moe_sort_padded: %d experts", experts);
    moe_sort_padded_kernel<<<1, 1024, 2 * experts * sizeof(int), (cudaStream_t)stream>>>(
        ids, num_pairs, experts, max_rows, row_pair, pos_of_pair, group_of_tile, tiles_m);
    return ti_check_launch("moe_sort_padded");
}

extern "C" int ti_moe_gather_scaled(const void* h, int h_stride, const int* row_pair, const int* tiles_m,
                                    const float* weights, int top, int width, int max_rows, void* a, void* stream) {
    TI_REQUIRE(width % 8 == 0 && h_stride % 8 == 0 && ((uintptr_t)h) % 16 == 0 && ((uintptr_t)a) % 16 == 0,
               "moe_gather_scaled: rows must be 16-byte aligned");
    if (max_rows == 0) return 0;
    moe_gather_scaled_kernel<<<max_rows, 128, 0, (cudaStream_t)stream>>>((const bf16*)h, h_stride, row_pair, tiles_m,
                                                                        weights, top, width, (bf16*)a);
    return ti_check_launch("moe_gather_scaled");
}

extern "C" int ti_moe_combine_rows(const float* rows, const int* pos_of_pair, int top, int width, int num_tokens,
                                   float* residual, int res_stride, const float* weights, const int* ids, int experts,
                                   const float* id_weights, const void* h, int h_stride, void* stream) {
    TI_REQUIRE(width % 4 == 0 && ((uintptr_t)rows) % 16 == 0, "moe_combine_rows: rows of four-float groups, 16-byte aligned");
    const size_t total = (size_t)num_tokens * (width / 4);
    if (total == 0) return 0;
    moe_combine_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        rows, pos_of_pair, top, width, num_tokens, residual, res_stride, weights, ids, experts, id_weights,
        (const bf16*)h, h_stride);
    return ti_check_launch("moe_combine_rows");
}

extern "C" int ti_moe_grouped_supported(int width, int ff, int experts) {
    return width % 32 == 0 && ff % 32 == 0 && experts >= 1 && experts <= 4096;
}

// Scratch the caller brings: sorted_slot int32 [pairs], tiles int32 [(pairs / 64 + experts) * 3],
// meta int32 [1], y_sorted bfloat16 [pairs, ff], out_rows float32 [pairs, width].
extern "C" int ti_moe_grouped(const void* h, int h_stride, const void* w_gate_up, int interleaved,
                              const void* w_down, const int* ids, const float* weights, int num_tokens,
                              int top, int experts, int width, int ff, int* sorted_slot, int* tiles,
                              int* meta, void* y_sorted, float* out_rows, float* residual,
                              int res_stride, int act, float act_limit, float act_alpha, int identity, void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(ti_moe_grouped_supported(width, ff, experts),
               "moe_grouped: width %d and expert size %d must be multiples of 32", width, ff);
    TI_REQUIRE(h_stride % 8 == 0 && ((uintptr_t)h) % 16 == 0, "moe_grouped: rows of h must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const int pairs = num_tokens * top;
    const int max_tiles = pairs / BM + experts;
    TI_REQUIRE(max_tiles <= 65535, "moe_grouped: %d tiles exceed the grid limit", max_tiles);
    moe_sort_kernel<<<1, 1024, 2 * experts * sizeof(int), s>>>(ids, pairs, experts, sorted_slot, tiles, meta);
    constexpr int SMEM = STAGES * STAGE_BYTES;
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e1 = cudaFuncSetAttribute(moe_grouped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        cudaError_t e2 = cudaFuncSetAttribute(moe_grouped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e1 != cudaSuccess || e2 != cudaSuccess) return ti_fail("moe_grouped: cannot set the shared memory size");
        configured.mark();
    }
    dim3 g1((ff + BNW / 2 - 1) / (BNW / 2), max_tiles);
    moe_grouped_kernel<true><<<g1, THREADS, SMEM, s>>>(
        (const bf16*)h, h_stride, sorted_slot, tiles, meta, top, (const bf16*)w_gate_up, interleaved, ff, width,
        weights, (bf16*)y_sorted, nullptr, act, act_limit, act_alpha);
    dim3 g2((width + BNW - 1) / BNW, max_tiles);
    moe_grouped_kernel<false><<<g2, THREADS, SMEM, s>>>(
        (const bf16*)y_sorted, ff, sorted_slot, tiles, meta, top, (const bf16*)w_down, 0, width, ff,
        nullptr, nullptr, out_rows, 0, 0.0f, 0.0f);
    const size_t total = (size_t)num_tokens * width;
    // `identity`: slots may name identity experts (an index not below `experts`)
    moe_combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(out_rows, top, width, num_tokens,
                                                                       residual, res_stride, identity ? ids : nullptr,
                                                                       experts, weights, (const bf16*)h, h_stride);
    return ti_check_launch("moe_grouped");
}
