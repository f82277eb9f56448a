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
    extern __shared__ float row_s[];          // q | k as float32, then cos | sin of the token's angles
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int q_width = p.q_heads * p.head_dim, k_width = p.kv_heads * p.head_dim, v_width = p.kv_heads * p.value_dim;
    const int pos = p.positions[t];
    const int page = p.block_table[(size_t)p.token_span[t] * p.table_stride + pos / p.page_tokens];
    if (page < 0 && threadIdx.x == 0) atomicExch(p.error_flag, 2);
    const float* row = p.proj + (size_t)t * p.proj_stride;
    float* qk = row_s;
    float* turn = row_s + q_width + k_width;
    const int half = p.frequencies ? p.rotary_dim >> 1 : 0;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * p.frequencies[i], &s, &c);
        turn[i] = c;
        turn[half + i] = s;
    }
    float q_squares = 0.0f, k_squares = 0.0f;
    for (int i = threadIdx.x; i < q_width + k_width; i += blockDim.x) {
        const float x = row[i] + (p.bias ? p.bias[i] : 0.0f);
        qk[i] = x;
        if (i < q_width) q_squares += x * x; else k_squares += x * x;
    }
    float q_factor = 1.0f, k_factor = 1.0f;
    if (p.q_norm_w) {
        q_factor = 1.0f / sqrtf(block_sum(q_squares, scratch) / (float)q_width + p.norm_eps);
        k_factor = 1.0f / sqrtf(block_sum(k_squares, scratch) / (float)k_width + p.norm_eps);
    }
    __syncthreads();
    if (p.q_norm_w) {
        for (int i = threadIdx.x; i < q_width + k_width; i += blockDim.x)
            qk[i] = i < q_width ? qk[i] * q_factor * p.q_norm_w[i] : qk[i] * k_factor * p.k_norm_w[i - q_width];
        __syncthreads();
    }
    if (half > 0) {
        const int heads = p.q_heads + p.kv_heads;             // k heads follow the q heads at the same head size
        for (int unit = threadIdx.x; unit < heads * half; unit += blockDim.x) {
            const int h = unit / half, i = unit - h * half;
            float* head = qk + (size_t)h * p.head_dim;
            const float u = head[i], v = head[i + half];
            head[i] = u * turn[i] - v * turn[half + i];
            head[i + half] = v * turn[i] + u * turn[half + i];
        }
        __syncthreads();
    }
    const float temperature = p.temp_every > 0
        ? 1.0f + p.temp_coef * logf((float)((pos + 1) / p.temp_every + 1)) : 1.0f;
    A* q_row = static_cast<A*>(p.q_out) + (size_t)t * p.q_stride;
    A* k_cache = static_cast<A*>(p.k_cache);
    A* v_cache = static_cast<A*>(p.v_cache);
    const long long in_page = pos % p.page_tokens;
    const int q_store = p.q_heads * p.key_store, k_store = p.kv_heads * p.key_store, v_store = p.kv_heads * p.value_store;
    for (int i = threadIdx.x; i < q_store + k_store + v_store; i += blockDim.x) {
        if (i < q_store) {
            const int head = i / p.key_store, e = i % p.key_store;
            q_row[i] = from_float<A>(e < p.head_dim ? qk[head * p.head_dim + e] * temperature : 0.0f);
        } else if (i < q_store + k_store) {
            if (page < 0) continue;
            const int j = i - q_store, head = j / p.key_store, e = j % p.key_store;
            k_cache[(long long)page * p.page_stride + ((long long)head * p.page_tokens + in_page) * p.key_store + e] =
                from_float<A>(e < p.head_dim ? qk[q_width + head * p.head_dim + e] : 0.0f);
        } else {
            const int j = i - q_store - k_store, head = j / p.value_store, e = j % p.value_store;
            float v = 0.0f;
            if (e < p.value_dim) {
                const int column = head * p.value_dim + e;
                const int src = q_width + k_width + column;
                v = row[src] + (p.bias ? p.bias[src] : 0.0f);
                if (p.blend == 1) p.first_values[(size_t)t * p.first_stride + column] = v;
                if (p.blend == 2) v = (1.0f - p.lam) * v + p.lam * p.first_values[(size_t)t * p.first_stride + column];
            }
            if (page >= 0)
                v_cache[(long long)page * p.value_page_stride +
                        ((long long)head * p.page_tokens + in_page) * p.value_store + e] = from_float<A>(v);
        }
    }
    (void)v_width;
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
    const size_t smem = ((size_t)(q_heads + kv_heads) * head_dim + (frequencies ? rotary_dim : 0)) * sizeof(float);
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
    if (act_dtype == kFloat32)
        launch_chained(qkv_prepare_kernel<float>, tokens, 256, smem, stream, args);
    else
        launch_chained(qkv_prepare_kernel<__nv_bfloat16>, tokens, 256, smem, stream, args);
    return check_launch("qkv_prepare");
}
