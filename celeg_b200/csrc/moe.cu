// Mixture of experts: router, grouping of (token, choice) pairs by expert, the experts' two products, and the
// weighted sum.
//
//   route      from z = W_r h (a product with float32 sums, made before): s = softmax(z) over all experts; the `top`
//              experts with the largest s + correction are chosen (ties: the lower index), their weights are
//              s / (sum of the chosen s + 1e-20); also the sigmoid of one more column of z, the gate of a shared
//              expert. One warp a token.
//   group      pairs (token, choice) ordered by expert: the source row of every place, the place of every pair,
//              and a table of row tiles (expert, first place, rows) for the products. One block, one launch;
//              the order inside an expert is not fixed, and no result depends on it.
//   expert product
//              out[place] = act(x[source(place)] . W_e^T) tile by tile over the table: 64 x 64 tiles, FFMA in
//              ascending k (float32 path) or warp-level 16 x 16 x 16 tensor-core tiles with float32 accumulators (bfloat16).
//              The grid is sized for the most tiles the step can have; blocks beyond the table leave at once,
//              so nothing about the launch depends on the routing (CUDA graphs replay it).
//   few pairs  out[pair] = act(x[token(pair)] . W_e^T) with a warp per output element row: the weights of the
//              chosen experts stream once, no grouping.
//   combine    y[t] = sum_k weight[t, k] out[place(t, k)] (+ gate[t] shared[t]), summed in the order of k.
#include <mma.h>

#include "common.cuh"

namespace celeg_b200 {

constexpr int kMoeTile = 64;

__device__ __forceinline__ float expert_activation(float z, int kind) {
    if (kind < 0) return z;
    return activate(z, kind);
}

// ------------------------------------------------------------------------------------------------ router
// logits: float32 [tokens, stride] = h W_r^T from a product with float32 sums (column `experts`, if asked for, is the
// shared expert's gate before its sigmoid). One warp a token: softmax over all experts, the choice, the weights.
__global__ void moe_route_kernel(const float* logits, int stride, const float* bias, const float* correction, int gate_column,
                                 int* chosen, float* weights, float* shared_gate, int tokens, int experts, int top) {
    extern __shared__ float route_smem[];          // per warp: scores [experts]
    chain_release();
    chain_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x * warps + warp;
    if (t >= tokens) return;
    float* scores = route_smem + (size_t)warp * experts;
    const float* row = logits + (size_t)t * stride;
    if (gate_column >= 0 && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-row[gate_column]));
    float largest = -INFINITY;
    // (a bias of the logits shifts choice and weights alike)
    for (int e = lane; e < experts; e += 32) largest = fmaxf(largest, row[e] + (bias ? bias[e] : 0.0f));
    largest = warp_max(largest);
    float total = 0.0f;
    for (int e = lane; e < experts; e += 32) {
        const float p = expf(row[e] + (bias ? bias[e] : 0.0f) - largest);
        scores[e] = p;
        total += p;
    }
    total = warp_sum(total);
    __syncwarp();
    for (int e = lane; e < experts; e += 32) scores[e] = scores[e] / total;
    __syncwarp();
    // the `top` largest of s + correction, one after the other; a taken expert is marked by a negative score
    // (scores are not negative)
    float picked_sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = experts;
        for (int e = lane; e < experts; e += 32) {
            const float s = scores[e];
            if (s < 0.0f) continue;
            const float c = s + (correction ? correction[e] : 0.0f);
            if (c > best) { best = c; best_e = e; }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_e = __shfl_xor_sync(0xffffffffu, best_e, offset);
            if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
        }
        if (best_e >= experts) best_e = 0;             // (not a number everywhere: keep the indices valid)
        const float s = fabsf(scores[best_e]);
        picked_sum += s;
        __syncwarp();
        if (lane == 0) {
            chosen[(size_t)t * top + k] = best_e;
            weights[(size_t)t * top + k] = s;
            scores[best_e] = -s - 1e-30f;
        }
        __syncwarp();
    }
    const float inv = 1.0f / (picked_sum + 1e-20f);
    for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= inv;
}

// ------------------------------------------------------------------------------------------------ grouping
// layout of `table` (int32): [0] number of tiles; then per tile (expert, first place, rows) from table[4] on
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* chosen, int pairs, int experts, int top,
                                                         int tile_rows, int* place_of_pair, int* source_of_place,
                                                         int* table) {
    extern __shared__ int group_smem[];            // counts [experts] | cursor [experts]
    chain_release();
    chain_wait();
    int* counts = group_smem;
    int* cursor = group_smem + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&counts[chosen[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            cursor[e] = at;
            for (int first = 0; first < counts[e]; first += tile_rows) {
                table[4 + 3 * tiles] = e;
                table[4 + 3 * tiles + 1] = at + first;
                table[4 + 3 * tiles + 2] = min(tile_rows, counts[e] - first);
                ++tiles;
            }
            at += counts[e];
        }
        table[0] = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int place = atomicAdd(&cursor[chosen[p]], 1);
        place_of_pair[p] = place;
        source_of_place[place] = p / top;
    }
}

// one block a place: a row copied in units of 16 bytes (or of one element, where rows are not aligned)
__global__ void moe_gather_rows_kernel(const unsigned char* x, long long x_stride_bytes, const int* source,
                                       unsigned char* out, long long out_stride_bytes, int bytes, int unit) {
    chain_release();
    chain_wait();
    const unsigned char* src = x + (long long)source[blockIdx.x] * x_stride_bytes;
    unsigned char* dst = out + (long long)blockIdx.x * out_stride_bytes;
    if (unit == 16) {
        for (int i = threadIdx.x * 16; i < bytes; i += blockDim.x * 16)
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (int i = threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
    }
}

// ------------------------------------------------------------------------------------------------ products
struct ExpertProductArgs {
    const void* x; int x_stride;                   // operand rows
    const int* source;                             // row of x for every place (null: the place itself)
    const void* weights; long long expert_stride; int w_stride;     // [experts][n][k]
    void* out; int out_stride;                     // [places, n]
    const int* table;
    int n, k, activation;                          // activation: a code of activate(), or -1 for none
};

template <typename A>
__global__ void __launch_bounds__(256) expert_product_ffma_kernel(const ExpertProductArgs a) {
    __shared__ float xs[16][kMoeTile + 4];
    __shared__ float ws[16][kMoeTile + 4];
    __shared__ int rows_of[kMoeTile];
    chain_release();
    chain_wait();
    const int tile = blockIdx.y;
    if (tile >= a.table[0]) return;
    const int expert = a.table[4 + 3 * tile], first = a.table[4 + 3 * tile + 1], rows = a.table[4 + 3 * tile + 2];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int col0 = blockIdx.x * kMoeTile;
    if (threadIdx.x < kMoeTile)
        rows_of[threadIdx.x] = threadIdx.x < rows ? (a.source ? a.source[first + threadIdx.x] : first + threadIdx.x) : -1;
    __syncthreads();
    const A* x = static_cast<const A*>(a.x);
    const A* w = static_cast<const A*>(a.weights) + (size_t)expert * a.expert_stride;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < a.k; k0 += 16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int src = rows_of[r], gc = col0 + r, gk = k0 + kk;
            xs[kk][r] = (src >= 0 && gk < a.k) ? to_float(x[(size_t)src * a.x_stride + gk]) : 0.0f;
            ws[kk][r] = (gc < a.n && gk < a.k) ? to_float(w[(size_t)gc * a.w_stride + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float xa[4], wb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xa[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wb[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xa[i], wb[j], acc[i][j]);
        }
        __syncthreads();
    }
    A* out = static_cast<A*>(a.out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc < a.n) out[(size_t)(first + r) * a.out_stride + gc] = from_float<A>(expert_activation(acc[i][j], a.activation));
        }
    }
}

// bfloat16 operands on the tensor cores: a 64 x 64 tile by 4 warps (each 32 x 32 as 2 x 2 fragments of 16 x 16),
// k in steps of 32 through shared memory; k must be a multiple of 8 (16-byte loads), anything else takes the
// FFMA kernel.
__global__ void __launch_bounds__(128) expert_product_mma_kernel(const ExpertProductArgs a) {
    using namespace nvcuda;
    constexpr int kDepth = 32, kPitch = kDepth + 8;
    __shared__ __align__(32) __nv_bfloat16 xs[kMoeTile][kPitch];
    __shared__ __align__(32) __nv_bfloat16 ws[kMoeTile][kPitch];
    __shared__ __align__(32) float cs[4][32][36];
    __shared__ int rows_of[kMoeTile];
    chain_release();
    chain_wait();
    const int tile = blockIdx.y;
    if (tile >= a.table[0]) return;
    const int expert = a.table[4 + 3 * tile], first = a.table[4 + 3 * tile + 1], rows = a.table[4 + 3 * tile + 2];
    const int col0 = blockIdx.x * kMoeTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x < kMoeTile)
        rows_of[threadIdx.x] = threadIdx.x < rows ? (a.source ? a.source[first + threadIdx.x] : first + threadIdx.x) : -1;
    __syncthreads();
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(a.x);
    const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(a.weights) + (size_t)expert * a.expert_stride;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[i][j], 0.0f);
    const int wr = (warp >> 1) * 32, wc = (warp & 1) * 32;
    for (int k0 = 0; k0 < a.k; k0 += kDepth) {
        // 64 rows x 32 k = 256 pieces of 8 elements for each operand: two a thread
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int piece = threadIdx.x + i * 128;
            const int r = piece >> 2, kk = (piece & 3) * 8;
            const int src = rows_of[r], gc = col0 + r, gk = k0 + kk;
            uint4 xv = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
            if (src >= 0 && gk < a.k) xv = *reinterpret_cast<const uint4*>(x + (size_t)src * a.x_stride + gk);
            if (gc < a.n && gk < a.k) wv = *reinterpret_cast<const uint4*>(w + (size_t)gc * a.w_stride + gk);
            *reinterpret_cast<uint4*>(&xs[r][kk]) = xv;
            *reinterpret_cast<uint4*>(&ws[r][kk]) = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kDepth; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa[2];
            wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) wmma::load_matrix_sync(fa[i], &xs[wr + 16 * i][kk], kPitch);
#pragma unroll
            for (int j = 0; j < 2; ++j) wmma::load_matrix_sync(fb[j], &ws[wc + 16 * j][kk], kPitch);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) wmma::mma_sync(acc[i][j], fa[i], fb[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) wmma::store_matrix_sync(&cs[warp][16 * i][16 * j], acc[i][j], 36, wmma::mem_row_major);
    __syncwarp();
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(a.out);
    for (int r = 0; r < 32; ++r) {
        const int row = wr + r, gc = col0 + wc + lane;
        if (row < rows && gc < a.n)
            out[(size_t)(first + row) * a.out_stride + gc] = __float2bfloat16_rn(expert_activation(cs[warp][r][lane], a.activation));
    }
}

// Few pairs: one warp per (pair, output element); the experts' matrices stream once each (pairs that chose the same
// expert meet in the L2).
template <typename A>
__global__ void expert_rows_kernel(const A* x, int x_stride, int pairs_per_row, const int* chosen, const A* weights,
                                   long long expert_stride, int w_stride, A* out, int out_stride, int pairs, int n, int k,
                                   int activation, int vectors) {
    chain_release();
    chain_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int j = blockIdx.x * warps + warp;
    const int pair = blockIdx.y;
    if (j >= n) return;
    const A* row = x + (size_t)(pair / pairs_per_row) * x_stride;
    const A* w = weights + (size_t)chosen[pair] * expert_stride + (size_t)j * w_stride;
    float sum = 0.0f;
    if (sizeof(A) == 2 && vectors) {
        // 8 elements a load, four loads of the weights in flight a lane
        const uint4* rv = reinterpret_cast<const uint4*>(row);
        const uint4* wv = reinterpret_cast<const uint4*>(w);
        const int pieces = k >> 3;
        float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int c0 = lane; c0 < pieces; c0 += 128) {
            uint4 wq[4], xq[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (c0 + 32 * u < pieces) { wq[u] = __ldg(wv + c0 + 32 * u); xq[u] = rv[c0 + 32 * u]; }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (c0 + 32 * u >= pieces) continue;
                const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wq[u]);
                const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xq[u]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 a = __bfloat1622float2(xh[i]), b = __bfloat1622float2(wh[i]);
                    part[u] = fmaf(a.x, b.x, part[u]);
                    part[u] = fmaf(a.y, b.y, part[u]);
                }
            }
        }
        sum = (part[0] + part[1]) + (part[2] + part[3]);
    } else {
        for (int c = lane; c < k; c += 32) sum = fmaf(to_float(row[c]), to_float(w[c]), sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) out[(size_t)pair * out_stride + j] = from_float<A>(expert_activation(sum, activation));
}

// ------------------------------------------------------------------------------------------------ combine
template <typename A>
__global__ void moe_combine_kernel(const A* expert_out, int out_stride, const int* place_of_pair, const float* weights,
                                   const A* shared, const float* shared_gate, A* y, int tokens, int width, int top) {
    chain_release();
    chain_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        const int pair = t * top + k;
        const int place = place_of_pair ? place_of_pair[pair] : pair;
        sum = fmaf(weights[pair], to_float(expert_out[(size_t)place * out_stride + c]), sum);
    }
    if (shared) sum = fmaf(shared_gate ? shared_gate[t] : 1.0f, to_float(shared[(size_t)t * width + c]), sum);
    y[(size_t)t * width + c] = from_float<A>(sum);
}

// bfloat16 rows whose width is a multiple of 8: 16 bytes a thread and row
__global__ void moe_combine_vec_kernel(const __nv_bfloat16* expert_out, int out_stride, const int* place_of_pair,
                                       const float* weights, const __nv_bfloat16* shared, const float* shared_gate,
                                       __nv_bfloat16* y, int tokens, int width, int top) {
    chain_release();
    chain_wait();
    const int pieces = width >> 3;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * pieces) return;
    const int t = (int)(i / pieces), c = (int)(i % pieces) << 3;
    float sum[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    auto add = [&](const __nv_bfloat16* row, float w) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(h[j]);
            sum[2 * j] = fmaf(w, v.x, sum[2 * j]);
            sum[2 * j + 1] = fmaf(w, v.y, sum[2 * j + 1]);
        }
    };
    for (int k = 0; k < top; ++k) {
        const int pair = t * top + k;
        add(expert_out + (size_t)(place_of_pair ? place_of_pair[pair] : pair) * out_stride, weights[pair]);
    }
    if (shared) add(shared + (size_t)t * width, shared_gate ? shared_gate[t] : 1.0f);
    uint4 packed;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(sum[2 * j], sum[2 * j + 1]);
    *reinterpret_cast<uint4*>(y + (size_t)t * width + c) = packed;
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_moe_route(const float* logits, int stride, const float* bias, const float* correction, int gate_column, int* chosen,
                              float* weights, float* shared_gate, int tokens, int experts, int top, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts && stride >= experts,
                  "moe_route: invalid sizes tokens=%d experts=%d top=%d stride=%d", tokens, experts, top, stride);
    CELEG_REQUIRE(experts <= 2048, "moe_route: %d experts exceed a block's shared memory", experts);
    CELEG_REQUIRE(gate_column < stride && (gate_column < 0 || shared_gate != nullptr),
                  "moe_route: the shared gate's column %d lies outside a row of %d, or has no output", gate_column, stride);
    if (tokens == 0) return 0;
    const int warps = 4;
    const size_t smem = (size_t)warps * experts * sizeof(float);
    const unsigned blocks = (unsigned)((tokens + warps - 1) / warps);
    launch_chained(moe_route_kernel, blocks, warps * 32, smem, stream, logits, stride, bias, correction, gate_column, chosen,
                   weights, shared_gate, tokens, experts, top);
    return check_launch("moe_route");
}

// table: int32 [4 + 3 * (pairs / tile_rows + experts)] at least; tile_rows: 64 for this file's products, 128 for the
// grouped tcgen05 product
CELEG_API int celeg_moe_group(const int* chosen, int tokens, int experts, int top, int tile_rows, int* place_of_pair,
                              int* source_of_place, int* table, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && experts <= 4096 && (tile_rows == kMoeTile || tile_rows == 128),
                  "moe_group: invalid sizes tokens=%d experts=%d top=%d tile_rows=%d", tokens, experts, top, tile_rows);
    if (tokens == 0) return 0;
    launch_chained(moe_group_kernel, 1, 1024, (size_t)2 * experts * sizeof(int), stream, chosen, tokens * top, experts,
                   top, tile_rows, place_of_pair, source_of_place, table);
    return check_launch("moe_group");
}

// out[place] = x[source[place]] for every place: the rows of a step ordered by expert, for a product that reads
// its operand by TMA
CELEG_API int celeg_moe_gather_rows(const void* x, int x_stride, const int* source, void* out, int out_stride, int places,
                                    int width, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(places >= 0 && width > 0, "moe_gather_rows: invalid sizes places=%d width=%d", places, width);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "moe_gather_rows: unknown dtype code %d", act_dtype);
    if (places == 0) return 0;
    const int bytes = width * (act_dtype == kFloat32 ? 4 : 2);
    const int unit = (bytes % 16 == 0 && ((size_t)x & 15) == 0 && ((size_t)out & 15) == 0 &&
                      (x_stride * (bytes / width)) % 16 == 0 && (out_stride * (bytes / width)) % 16 == 0) ? 16 : (bytes / width);
    launch_chained(moe_gather_rows_kernel, places, 128, 0, stream, (const unsigned char*)x,
                   (long long)x_stride * (bytes / width), source, (unsigned char*)out, (long long)out_stride * (bytes / width),
                   bytes, unit);
    return check_launch("moe_gather_rows");
}

// out[place, :n] = act(x[source[place]] . W[expert of the place's tile]^T); max_tiles bounds the table's tiles
CELEG_API int celeg_expert_product(const void* x, int x_stride, const int* source, const void* weights,
                                   long long expert_stride, int w_stride, void* out, int out_stride, const int* table,
                                   int max_tiles, int n, int k, int activation, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(max_tiles >= 0 && n > 0 && k > 0 && activation >= -1 && activation <= 3,
                  "expert_product: invalid sizes tiles=%d n=%d k=%d activation=%d", max_tiles, n, k, activation);
    CELEG_REQUIRE(max_tiles <= 65535, "expert_product: %d tiles exceed one launch", max_tiles);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "expert_product: unknown dtype code %d", act_dtype);
    if (max_tiles == 0) return 0;
    const ExpertProductArgs args = {x, x_stride, source, weights, expert_stride, w_stride, out, out_stride, table, n, k,
                                    activation};
    dim3 grid((n + kMoeTile - 1) / kMoeTile, max_tiles);
    if (act_dtype == kFloat32) {
        launch_chained(expert_product_ffma_kernel<float>, grid, 256, 0, stream, args);
    } else if (k % 8 == 0 && x_stride % 8 == 0 && w_stride % 8 == 0 && expert_stride % 8 == 0 &&
               (((size_t)x | (size_t)weights) & 15) == 0) {
        launch_chained(expert_product_mma_kernel, grid, 128, 0, stream, args);
    } else {
        launch_chained(expert_product_ffma_kernel<__nv_bfloat16>, grid, 256, 0, stream, args);
    }
    return check_launch("expert_product");
}

// out[pair, :n] = act(x[pair / pairs_per_row] . W[chosen[pair]]^T), for few pairs
CELEG_API int celeg_expert_rows(const void* x, int x_stride, int pairs_per_row, const int* chosen, const void* weights,
                                long long expert_stride, int w_stride, void* out, int out_stride, int pairs, int n, int k,
                                int activation, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(pairs >= 0 && pairs <= 65535 && n > 0 && k > 0 && pairs_per_row > 0 && activation >= -1 && activation <= 3,
                  "expert_rows: invalid sizes pairs=%d n=%d k=%d activation=%d", pairs, n, k, activation);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "expert_rows: unknown dtype code %d", act_dtype);
    if (pairs == 0) return 0;
    const int warps = 8;
    dim3 grid((n + warps - 1) / warps, pairs);
    const int vectors = k % 8 == 0 && x_stride % 8 == 0 && w_stride % 8 == 0 && expert_stride % 8 == 0 &&
                        (((size_t)x | (size_t)weights) & 15) == 0;
    if (act_dtype == kFloat32)
        launch_chained(expert_rows_kernel<float>, grid, warps * 32, 0, stream, (const float*)x, x_stride, pairs_per_row,
                       chosen, (const float*)weights, expert_stride, w_stride, (float*)out, out_stride, pairs, n, k,
                       activation, 0);
    else
        launch_chained(expert_rows_kernel<__nv_bfloat16>, grid, warps * 32, 0, stream, (const __nv_bfloat16*)x, x_stride,
                       pairs_per_row, chosen, (const __nv_bfloat16*)weights, expert_stride, w_stride, (__nv_bfloat16*)out,
                       out_stride, pairs, n, k, activation, vectors);
    return check_launch("expert_rows");
}

CELEG_API int celeg_moe_combine(const void* expert_out, int out_stride, const int* place_of_pair, const float* weights,
                                const void* shared, const float* shared_gate, void* y, int tokens, int width, int top,
                                int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && width > 0 && top > 0, "moe_combine: invalid sizes tokens=%d width=%d top=%d", tokens,
                  width, top);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "moe_combine: unknown dtype code %d", act_dtype);
    if (tokens == 0) return 0;
    const long long units = (long long)tokens * width;
    const unsigned blocks = (unsigned)((units + 255) / 256);
    if (act_dtype == kBFloat16 && width % 8 == 0 && out_stride % 8 == 0 &&
        (((size_t)expert_out | (size_t)shared | (size_t)y) & 15) == 0) {
        const unsigned vec_blocks = (unsigned)((units / 8 + 255) / 256);
        launch_chained(moe_combine_vec_kernel, vec_blocks, 256, 0, stream, (const __nv_bfloat16*)expert_out, out_stride,
                       place_of_pair, weights, (const __nv_bfloat16*)shared, shared_gate, (__nv_bfloat16*)y, tokens, width,
                       top);
        return check_launch("moe_combine");
    }
    if (act_dtype == kFloat32)
        launch_chained(moe_combine_kernel<float>, blocks, 256, 0, stream, (const float*)expert_out, out_stride,
                       place_of_pair, weights, (const float*)shared, shared_gate, (float*)y, tokens, width, top);
    else
        launch_chained(moe_combine_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)expert_out,
                       out_stride, place_of_pair, weights, (const __nv_bfloat16*)shared, shared_gate, (__nv_bfloat16*)y,
                       tokens, width, top);
    return check_launch("moe_combine");
}
