// Latent attention: what stands between its projections and the attention kernels.
//
// Per position the mixer caches ONE vector [c | r]: c, the RMS-normalised low-rank vector that every head's key
// and value are up-projections of (k_h = U_h c, v_h = V_h c), and r, a rotated key part shared by all heads.
// Because a head's score is q_h . (U_h c) + q_rot_h . r = (U_h^T q_h) . c + q_rot_h . r, the query is taken
// to the latent space once per token ("absorbed"), the attention runs over the cached vectors as they are, as
// one key head of size rank + rot that all query heads share and whose first `rank` elements are also the
// value, and the head's output V_h (sum_j p_j c_j) is up-projected afterwards. Nothing per head is ever cached
// or rebuilt from the cache.
//
//   latent_prepare   c = rms_norm(down[:rank]) * w -> cache;  r = rotate(down[rank:]) -> cache;
//                    rotate(q_h[dim:]) -> absorbed query [.., rank:]
//   head_project     out[t, h, :] = in[t, h, :] . M_h for a matrix per head taken out of a stored [out, in]
//                    projection (either orientation), optionally times sigmoid(gate[t, h]) or, with a gate per
//                    output element, sigmoid(gate[t, h, n]):
//                    the absorption (U_h^T q_h) and the value up-projection with the head's output gate
//
// Rotation: dimensions (2i, 2i + 1) form a pair (or, where asked for, i and i + half of the rotated dimensions),
// angle = position x frequency_i (frequencies come scaled from the host), cos and sin times `magnitude`. Sums, norms and angles are float32; cache and query have the activation type.
#include "common.cuh"

namespace celeg_b200 {

struct LatentPrepareArgs {
    const void* q; int q_stride;              // [tokens, heads * (dim + rot)]
    const void* down; int down_stride;        // [tokens, rank + rot]
    const float* norm_weight;                 // [rank]
    const float* frequencies;                 // [rot / 2]
    float magnitude, eps;
    const int* positions; const int* token_span; const int* block_table; int table_stride;
    void* cache; long long page_stride; int page_tokens;     // pages of [page_tokens, rank + rot]
    void* query; int query_stride;            // [tokens, heads * (rank + rot)]: the rotated part is written here
    int heads, dim, rot, rotated, rank;      // rot: width of the rotated part; rotated <= rot: how much of it turns
    int halves;                               // pairs are (i, i + rotated / 2) instead of neighbours (2i, 2i + 1)
    int* error_flag;
};

template <typename A>
__global__ void latent_prepare_kernel(const LatentPrepareArgs a) {
    __shared__ float scratch[33];
    extern __shared__ float turn[];           // cos | sin of the token's angles, [rot / 2] each
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int pos = a.positions[t];
    const int half = a.rotated >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * a.frequencies[i], &s, &c);
        turn[i] = c * a.magnitude;
        turn[half + i] = s * a.magnitude;
    }
    const A* down = static_cast<const A*>(a.down) + (size_t)t * a.down_stride;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        const float x = to_float(down[i]);
        sum += x * x;
    }
    sum = block_sum(sum, scratch);            // (also orders the writes of `turn` before its reads)
    const float inv = 1.0f / sqrtf(sum / (float)a.rank + a.eps);
    const int page = a.block_table[(size_t)a.token_span[t] * a.table_stride + pos / a.page_tokens];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(a.error_flag, 2);
    } else {
        A* dst = static_cast<A*>(a.cache) + (size_t)page * a.page_stride + (size_t)(pos % a.page_tokens) * (a.rank + a.rot);
        for (int i = threadIdx.x; i < a.rank; i += blockDim.x)
            dst[i] = from_float<A>(to_float(down[i]) * inv * a.norm_weight[i]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int first = a.halves ? i : 2 * i, second = a.halves ? i + half : 2 * i + 1;
            const float u = to_float(down[a.rank + first]), v = to_float(down[a.rank + second]);
            dst[a.rank + first] = from_float<A>(u * turn[i] - v * turn[half + i]);
            dst[a.rank + second] = from_float<A>(v * turn[i] + u * turn[half + i]);
        }
        for (int i = a.rotated + threadIdx.x; i < a.rot; i += blockDim.x) dst[a.rank + i] = down[a.rank + i];
    }
    const A* q = static_cast<const A*>(a.q) + (size_t)t * a.q_stride;
    A* query = static_cast<A*>(a.query) + (size_t)t * a.query_stride;
    for (int unit = threadIdx.x; unit < a.heads * half; unit += blockDim.x) {
        const int h = unit / half, i = unit - h * half;
        const A* src = q + (size_t)h * (a.dim + a.rot) + a.dim;
        A* dst = query + (size_t)h * (a.rank + a.rot) + a.rank;
        const int first = a.halves ? i : 2 * i, second = a.halves ? i + half : 2 * i + 1;
        const float u = to_float(src[first]), v = to_float(src[second]);
        dst[first] = from_float<A>(u * turn[i] - v * turn[half + i]);
        dst[second] = from_float<A>(v * turn[i] + u * turn[half + i]);
    }
    const int rest = a.rot - a.rotated;
    for (int unit = threadIdx.x; unit < a.heads * rest; unit += blockDim.x) {
        const int h = unit / rest, i = a.rotated + unit % rest;
        query[(size_t)h * (a.rank + a.rot) + a.rank + i] = q[(size_t)h * (a.dim + a.rot) + a.dim + i];
    }
}

// out[t, h * out_head + n] = (sum_k in[t, h * in_head + k] * M[h * m_head + k * m_k + n * m_n]) (* sigmoid(gate[t, h]))
// for n < N, k < K: a matrix per head, read out of a stored projection with strides. 64 x 64 tiles of (tokens,
// outputs), FFMA in ascending k: an output's sum does not depend on the rows beside it.
struct HeadProjectArgs {
    const void* in; int in_stride, in_head;
    const void* matrix; long long m_head, m_k, m_n;
    void* out; int out_stride, out_head;
    const void* gate; int gate_stride;        // activation type [tokens, heads * gate_width] or null
    int gate_width;                           // 1: a gate per head; n: a gate per output element
    int tokens, n, k;
};

template <typename A>
__global__ void __launch_bounds__(256) head_project_kernel(const HeadProjectArgs a) {
    constexpr int kTile = 64, kDepth = 16;
    __shared__ float xs[kDepth][kTile + 4];
    __shared__ float ms[kDepth][kTile + 4];
    chain_release();
    chain_wait();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int head = blockIdx.z;
    const int row0 = blockIdx.y * kTile, col0 = blockIdx.x * kTile;
    const A* in = static_cast<const A*>(a.in) + (size_t)head * a.in_head;
    const A* matrix = static_cast<const A*>(a.matrix) + (size_t)head * a.m_head;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < a.k; k0 += kDepth) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            // operand rows: the 16 k of a row are neighbours in memory
            const int r = idx >> 4, kk = idx & 15;
            const int gr = row0 + r, gk = k0 + kk;
            xs[kk][r] = (gr < a.tokens && gk < a.k) ? to_float(in[(size_t)gr * a.in_stride + gk]) : 0.0f;
            // the matrix: whichever of k and n is contiguous runs along the threads
            int mk, mn;
            if (a.m_k == 1) { mk = idx & 15; mn = idx >> 4; } else { mn = idx & 63; mk = idx >> 6; }
            const int gn = col0 + mn, gmk = k0 + mk;
            ms[mk][mn] = (gn < a.n && gmk < a.k) ? to_float(matrix[(size_t)gmk * a.m_k + (size_t)gn * a.m_n]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kDepth; ++kk) {
            float x[4], m[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) m[j] = ms[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(x[i], m[j], acc[i][j]);
        }
        __syncthreads();
    }
    A* out = static_cast<A*>(a.out) + (size_t)head * a.out_head;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= a.tokens) continue;
        const A* gate = a.gate ? static_cast<const A*>(a.gate) + (size_t)gr * a.gate_stride + (size_t)head * a.gate_width
                               : nullptr;
        float factor = 1.0f;
        if (gate && a.gate_width == 1) factor = 1.0f / (1.0f + expf(-to_float(gate[0])));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc >= a.n) continue;
            if (gate && a.gate_width > 1) factor = 1.0f / (1.0f + expf(-to_float(gate[gc])));
            out[(size_t)gr * a.out_stride + gc] = from_float<A>(acc[i][j] * factor);
        }
    }
}

// rows of [heads, width] scaled in place by sigmoid(gate[t, h]): the head gate after a library product
template <typename A>
__global__ void head_gate_kernel(A* values, int stride, int head_width, const A* gate, int gate_stride, int tokens,
                                 int heads) {
    chain_release();
    chain_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long per_row = (long long)heads * head_width;
    if (i >= tokens * per_row) return;
    const int t = (int)(i / per_row), c = (int)(i % per_row);
    const float g = 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + c / head_width])));
    A* cell = values + (size_t)t * stride + c;
    *cell = from_float<A>(to_float(*cell) * g);
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_latent_prepare(const void* q, int q_stride, const void* down, int down_stride,
                                   const float* norm_weight, const float* frequencies, float magnitude, float eps,
                                   const int* positions, const int* token_span, const int* block_table,
                                   int table_stride, void* cache, long long page_stride, int page_tokens, void* query,
                                   int query_stride, int tokens, int heads, int dim, int rot, int rotated, int rank, int halves,
                                   int* error_flag, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && heads > 0 && dim >= 0 && rot >= 0 && rotated >= 0 && rotated <= rot && rotated % 2 == 0 &&
                  rank > 0 && page_tokens > 0 && eps > 0.0f,
                  "latent_prepare: invalid sizes tokens=%d heads=%d dim=%d rot=%d rotated=%d rank=%d page_tokens=%d",
                  tokens, heads, dim, rot, rotated, rank, page_tokens);
    CELEG_REQUIRE(rot <= 8192, "latent_prepare: %d rotated dimensions exceed a block's shared memory", rot);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "latent_prepare: unknown dtype code %d", act_dtype);
    if (tokens == 0) return 0;
    const LatentPrepareArgs args = {q, q_stride, down, down_stride, norm_weight, frequencies, magnitude, eps, positions,
                                    token_span, block_table, table_stride, cache, page_stride, page_tokens, query,
                                    query_stride, heads, dim, rot, rotated, rank, halves, error_flag};
    const size_t smem = (size_t)(rotated + 2) * sizeof(float);
    if (act_dtype == kFloat32)
        launch_chained(latent_prepare_kernel<float>, tokens, 128, smem, stream, args);
    else
        launch_chained(latent_prepare_kernel<__nv_bfloat16>, tokens, 128, smem, stream, args);
    return check_launch("latent_prepare");
}

CELEG_API int celeg_head_project(const void* in, int in_stride, int in_head, const void* matrix, long long m_head,
                                 long long m_k, long long m_n, void* out, int out_stride, int out_head, const void* gate,
                                 int gate_stride, int gate_width, int tokens, int heads, int n, int k, int act_dtype,
                                 cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && heads > 0 && n > 0 && k > 0 && (m_k == 1 || m_n == 1),
                  "head_project: invalid sizes tokens=%d heads=%d n=%d k=%d m_k=%lld m_n=%lld", tokens, heads, n, k, m_k,
                  m_n);
    CELEG_REQUIRE(!gate || gate_width == 1 || gate_width == n, "head_project: a gate of %d numbers for a head of %d outputs",
                  gate_width, n);
    CELEG_REQUIRE(heads <= 65535 && (tokens + 63) / 64 <= 65535, "head_project: %d heads or %d tokens exceed one launch",
                  heads, tokens);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "head_project: unknown dtype code %d", act_dtype);
    if (tokens == 0) return 0;
    const HeadProjectArgs args = {in, in_stride, in_head, matrix, m_head, m_k, m_n, out, out_stride, out_head, gate,
                                  gate_stride, gate_width, tokens, n, k};
    dim3 grid((n + 63) / 64, (tokens + 63) / 64, heads);
    if (act_dtype == kFloat32)
        launch_chained(head_project_kernel<float>, grid, 256, 0, stream, args);
    else
        launch_chained(head_project_kernel<__nv_bfloat16>, grid, 256, 0, stream, args);
    return check_launch("head_project");
}

CELEG_API int celeg_head_gate(void* values, int stride, int head_width, const void* gate, int gate_stride, int tokens,
                              int heads, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && heads > 0 && head_width > 0, "head_gate: invalid sizes tokens=%d heads=%d width=%d",
                  tokens, heads, head_width);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "head_gate: unknown dtype code %d", act_dtype);
    if (tokens == 0) return 0;
    const long long units = (long long)tokens * heads * head_width;
    const unsigned blocks = (unsigned)((units + 255) / 256);
    if (act_dtype == kFloat32)
        launch_chained(head_gate_kernel<float>, blocks, 256, 0, stream, (float*)values, stride, head_width,
                       (const float*)gate, gate_stride, tokens, heads);
    else
        launch_chained(head_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)values, stride,
                       head_width, (const __nv_bfloat16*)gate, gate_stride, tokens, heads);
    return check_launch("head_gate");
}
