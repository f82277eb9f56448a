// What stands between an attention mixer's fused [q | k | v] projection (float32 sums) and the paged attention
// kernels, for mixers that need more than a bias: one block a token does, in float32 and in this order,
//
//   1. the biases of q, k and v (optional);
//   2. one RMS norm over the whole q projection and one over the whole k projection, each with a weight as wide as
//      the projection (optional): x / sqrt(mean(x^2) + eps) * w, the mean over all heads' entries together;
//   3. the rotation of the first `rotary_dim` entries of every q and k head in pairs (i, i + rotary_dim / 2) by the
//      angle position * frequency_i (optional; frequencies come from the host, already divided by what the
//      configuration scales them by);
//   4. a factor on q that grows with the position: 1 + coef * ln(floor((position + 1) / every) + 1) (optional);
//   5. the blend of the values with those an earlier layer made of the same token: v <- (1 - lam) v + lam v_first
//      (`blend` 2), or the note of this layer's values for later layers (`blend` 1: v_first <- v);
//
// rounds once, and writes q to its buffer and k and v to the token's place in the paged cache. A stored head may be
// wider than the projected one (keys and values brought to one size for kernels that want them alike): the tail is
// zeros, which change no score and no result.
#include "common.cuh"

namespace celeg_b200 {

struct QkvPrepareArgs {
    const float* proj; int proj_stride;       // rows [q heads | k heads | v heads | ...] as projected, float32
    const float* bias;                        // q, k and v biases one after the other, or null
    const float* q_norm_w; const float* k_norm_w;      // [q width], [k width], or null (both or none)
    float norm_eps;
    const float* frequencies; int rotary_dim; // [rotary_dim / 2] or null
    float temp_coef; int temp_every;          // every <= 0: no factor
    int blend; float lam; float* first_values; int first_stride;     // [tokens, kv_heads * value_dim] float32
    void* q_out; int q_stride;                // queries in the activation type, head h at h * key_store
    const int* positions; const int* token_span; const int* block_table; int table_stride;
    void* k_cache; void* v_cache; long long page_stride, value_page_stride;
    int q_heads, kv_heads, head_dim, value_dim;    // sizes as projected
    int key_store, value_store;                    // sizes as stored
    int page_tokens;
    int* error_flag;
};

template <typename A>
__global__ void qkv_prepare_kernel(const QkvPrepareArgs p) {
    __shared__ float scratch[33];
    extern __shared__ __align__(16) float row_s[];       // q | k | v as float32, the first values, cos | sin of the angles
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int q_width = p.q_heads * p.head_dim, k_width = p.kv_heads * p.head_dim;
    const int qk_width = q_width + k_width;
    // (the token's position and span are asked for first and used last: the row's loads do not wait for them, and
    // the page's number, which hangs on both, is under way while the angles are made)
    const int pos = p.positions[t];
    const int span = p.token_span[t];
    const float* row = p.proj + (size_t)t * p.proj_stride;
    const int v_width = p.kv_heads * p.value_dim;
    const int row_width = qk_width + v_width;
    float* qk = row_s;                                    // q | k | v, biases added
    float* first_s = row_s + ((row_width + 3) & ~3);      // the first values of this token (blend 2)
    float* turn = first_s + (p.blend == 2 ? ((v_width + 3) & ~3) : 0);
    const int half = p.frequencies ? p.rotary_dim >> 1 : 0;
    const float* first_row = p.blend == 2 ? p.first_values + (size_t)t * p.first_stride : nullptr;
    // The row with its biases into shared memory, and the squares of q and of k. Four at a time where the rows allow
    // it, and then every load of a thread is under way before the first is used: a block's time is the time of its
    // chains of dependent loads.
    float q_squares = 0.0f, k_squares = 0.0f;
    const bool by_four = ((row_width | qk_width | q_width | p.proj_stride) & 3) == 0 && ((size_t)p.proj & 15) == 0 &&
                         ((size_t)p.bias & 15) == 0;
    if (by_four) {
        constexpr int kAhead = 4;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const float4* bias4 = reinterpret_cast<const float4*>(p.bias);
        const int quads = row_width >> 2;
        for (int base = threadIdx.x; base < quads; base += kAhead * blockDim.x) {
            float4 x[kAhead];
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int i = base + u * blockDim.x;
                x[u] = i < quads ? row4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int i = base + u * blockDim.x;
                if (i >= quads) continue;
                if (bias4) {
                    const float4 b = __ldg(bias4 + i);
                    x[u].x += b.x; x[u].y += b.y; x[u].z += b.z; x[u].w += b.w;
                }
                reinterpret_cast<float4*>(qk)[i] = x[u];
                const float squares = x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
                if (4 * i < q_width) q_squares += squares; else if (4 * i < qk_width) k_squares += squares;
            }
        }
    } else {
        for (int i = threadIdx.x; i < row_width; i += blockDim.x) {
            const float x = row[i] + (p.bias ? p.bias[i] : 0.0f);
            qk[i] = x;
            if (i < q_width) q_squares += x * x; else if (i < qk_width) k_squares += x * x;
        }
    }
    if (first_row)
        for (int i = threadIdx.x; i < v_width; i += blockDim.x) first_s[i] = first_row[i];
    const int page = p.block_table[(size_t)span * p.table_stride + pos / p.page_tokens];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * p.frequencies[i], &s, &c);
        turn[i] = c;
        turn[half + i] = s;
    }
    float q_factor = 1.0f, k_factor = 1.0f;
    if (p.q_norm_w) {
        q_factor = 1.0f / sqrtf(block_sum(q_squares, scratch) / (float)q_width + p.norm_eps);
        k_factor = 1.0f / sqrtf(block_sum(k_squares, scratch) / (float)k_width + p.norm_eps);
    }
    __syncthreads();
    const float temperature = p.temp_every > 0
        ? 1.0f + p.temp_coef * logf((float)((pos + 1) / p.temp_every + 1)) : 1.0f;
    A* q_row = static_cast<A*>(p.q_out) + (size_t)t * p.q_stride;
    const long long in_page = pos % p.page_tokens;
    if (page < 0 && threadIdx.x == 0) atomicExch(p.error_flag, 2);
    // a warp a head: norm scale, rotation, the query factor and the store in one pass over shared memory
    for (int unit = warp; unit < p.q_heads + p.kv_heads; unit += warps) {
        const bool is_q = unit < p.q_heads;
        if (!is_q && page < 0) continue;
        const float* head = qk + (size_t)unit * p.head_dim;
        const float* weight = !p.q_norm_w ? nullptr
                              : (is_q ? p.q_norm_w + (size_t)unit * p.head_dim
                                      : p.k_norm_w + (size_t)(unit - p.q_heads) * p.head_dim);
        const float factor = is_q ? q_factor : k_factor;
        const float after = is_q ? temperature : 1.0f;
        A* dst = is_q ? q_row + (size_t)unit * p.key_store
                      : static_cast<A*>(p.k_cache) + (long long)page * p.page_stride +
                            ((long long)(unit - p.q_heads) * p.page_tokens + in_page) * p.key_store;
        for (int i = lane; i < half; i += 32) {
            float u = head[i] * factor, v = head[i + half] * factor;
            if (weight) {
                u *= weight[i];
                v *= weight[i + half];
            }
            dst[i] = from_float<A>((u * turn[i] - v * turn[half + i]) * after);
            dst[i + half] = from_float<A>((v * turn[i] + u * turn[half + i]) * after);
        }
        for (int e = 2 * half + lane; e < p.head_dim; e += 32)
            dst[e] = from_float<A>(head[e] * factor * (weight ? weight[e] : 1.0f) * after);
        for (int e = p.head_dim + lane; e < p.key_store; e += 32) dst[e] = from_float<A>(0.0f);
    }
    for (int unit = warp; unit < p.kv_heads; unit += warps) {
        A* dst = page < 0 ? nullptr
                          : static_cast<A*>(p.v_cache) + (long long)page * p.value_page_stride +
                                ((long long)unit * p.page_tokens + in_page) * p.value_store;
        for (int e = lane; e < p.value_store; e += 32) {
            float v = 0.0f;
            if (e < p.value_dim) {
                const int column = unit * p.value_dim + e;
                v = qk[qk_width + column];
                if (p.blend == 1) p.first_values[(size_t)t * p.first_stride + column] = v;
                if (p.blend == 2) v = (1.0f - p.lam) * v + p.lam * first_s[column];
            }
            if (dst) dst[e] = from_float<A>(v);
        }
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_qkv_prepare(const float* proj, int proj_stride, const float* bias, const float* q_norm_w,
                                const float* k_norm_w, float norm_eps, const float* frequencies, int rotary_dim,
                                float temp_coef, int temp_every, int blend, float lam, float* first_values,
                                int first_stride, void* q_out, int q_stride, const int* positions, const int* token_span,
                                const int* block_table, int table_stride, void* k_cache, void* v_cache,
                                long long page_stride, long long value_page_stride, int tokens, int q_heads, int kv_heads,
                                int head_dim, int value_dim, int key_store, int value_store, int page_tokens,
                                int* error_flag, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && value_dim > 0 && page_tokens > 0 &&
                  key_store >= head_dim && value_store >= value_dim && q_stride >= q_heads * key_store &&
                  proj_stride >= q_heads * head_dim + kv_heads * (head_dim + value_dim),
                  "qkv_prepare: invalid sizes tokens=%d q_heads=%d kv_heads=%d head_dim=%d value_dim=%d stored %d / %d "
                  "strides %d / %d", tokens, q_heads, kv_heads, head_dim, value_dim, key_store, value_store, proj_stride,
                  q_stride);
    CELEG_REQUIRE((q_norm_w == nullptr) == (k_norm_w == nullptr) && (!q_norm_w || norm_eps > 0.0f),
                  "qkv_prepare: the whole-projection norm needs both weights and a positive eps");
    CELEG_REQUIRE(!frequencies || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim),
                  "qkv_prepare: %d rotated dimensions of a head of %d", rotary_dim, head_dim);
    CELEG_REQUIRE(blend == 0 || ((blend == 1 || blend == 2) && first_values && first_stride >= kv_heads * value_dim),
                  "qkv_prepare: blend %d without a place for the first values (stride %d)", blend, first_stride);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "qkv_prepare: unknown dtype code %d", act_dtype);
    if (tokens == 0) return 0;
    const size_t row_floats = ((size_t)(q_heads + kv_heads) * head_dim + (size_t)kv_heads * value_dim + 3) & ~(size_t)3;
    const size_t first_floats = blend == 2 ? (((size_t)kv_heads * value_dim + 3) & ~(size_t)3) : 0;
    const size_t smem = (row_floats + first_floats + (frequencies ? rotary_dim : 0)) * sizeof(float);
    CELEG_REQUIRE(smem <= 200 * 1024, "qkv_prepare: a row of %zu bytes exceeds a block's shared memory", smem);
    const QkvPrepareArgs args = {proj, proj_stride, bias, q_norm_w, k_norm_w, norm_eps, frequencies, rotary_dim,
                                 temp_coef, temp_every, blend, lam, first_values, first_stride, q_out, q_stride,
                                 positions, token_span, block_table, table_stride, k_cache, v_cache, page_stride,
                                 value_page_stride, q_heads, kv_heads, head_dim, value_dim, key_store, value_store,
                                 page_tokens, error_flag};
    cudaError_t status = cudaSuccess;
    if (smem > 40 * 1024) {
        status = act_dtype == kFloat32
            ? cudaFuncSetAttribute(qkv_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
            : cudaFuncSetAttribute(qkv_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) {
            set_error("qkv_prepare: %s", cudaGetErrorString(status));
            return -2;
        }
    }
    // A block's time is a chain of dependent loads (position, span, page) and two passes over a short row: more and
    // smaller blocks an SM hide it better than wide ones (2,048 tokens of 16 + 4 heads of 64: 20 us with 256 threads).
    const int threads = (q_heads + kv_heads) * head_dim <= 4096 ? 128 : 256;
    if (act_dtype == kFloat32)
        launch_chained(qkv_prepare_kernel<float>, tokens, threads, smem, stream, args);
    else
        launch_chained(qkv_prepare_kernel<__nv_bfloat16>, tokens, threads, smem, stream, args);
    return check_launch("qkv_prepare");
}
