// Paged causal grouped-query attention, general form: any head size, float32 or bfloat16 cache,
// any mix of spans. One warp per (query token, query head); the 32 lanes take 32 keys at a time
// for the scores and split the head dimension for the weighted sum of values; softmax is online
// (running maximum and denominator) in float32. A token's result depends only on its own keys,
// read in position order, so it is the same bit for bit however the batch was cut.
//
// Values may have another size than keys (``value_dim``), and instead of a window of recent positions a query may be
// limited to the keys of its own chunk of ``chunk`` positions, chunks counted from position 0 of the sequence.
//
// An optional table per query head of numbers by distance (query position minus key position, the last entry for
// everything farther) is added to the scaled scores.
//
// An optional sink per query head (a learned score that enters the denominator once, unscaled, with no
// value) is where the running maximum and denominator start.
//
// This is the whole attention of the float32 path and the fall-back of the bfloat16 path for
// head sizes the tensor-core kernels refuse.
//
// Counterpart in celeg: gqa_decode_paged_batch_kernel (src/backend/cuda/kernels/attention_paged.cuh:3-166),
// one block of 64 threads per (row, head) walking the keys one by one.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kAccRegs = 16;     // value_dim <= 32 * kAccRegs

template <typename A>
__global__ void attention_generic_kernel(const A* __restrict__ q, int q_row_stride, A* __restrict__ out,
                                         const A* __restrict__ k_cache, const A* __restrict__ v_cache,
                                         long long page_stride, long long value_page_stride,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ token_span,
                                         const int* __restrict__ block_table, int table_stride, int tokens,
                                         int q_heads, int kv_heads, int head_dim, int value_dim, int page_tokens,
                                         int window, int chunk, float scale, const float* __restrict__ sinks,
                                         const float* __restrict__ distance_bias, int distance_last,
                                         int* __restrict__ error_flag) {
    extern __shared__ float q_smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const long long unit = (long long)blockIdx.x * warps + warp;
    if (unit >= (long long)tokens * q_heads) return;
    const int t = (int)(unit / q_heads);
    const int h = (int)(unit % q_heads);
    const int kvh = h / (q_heads / kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_span[t] * table_stride;
    float* qs = q_smem + warp * head_dim;
    const A* qv = q + (size_t)t * q_row_stride + (size_t)h * head_dim;
    for (int i = lane; i < head_dim; i += 32) qs[i] = to_float(qv[i]) * scale;
    __syncwarp();

    float acc[kAccRegs];
#pragma unroll
    for (int r = 0; r < kAccRegs; ++r) acc[r] = 0.0f;
    // a sink is a score without key or value: the softmax starts from it (weight 1 at the maximum so far)
    float running_max = sinks ? sinks[h] : -INFINITY;
    float denom = sinks ? 1.0f : 0.0f;
    const int first_key = chunk > 0 ? (pos / chunk) * chunk : (window > 0 ? max(0, pos - window + 1) : 0);

    for (int base = first_key; base <= pos; base += 32) {
        const int key = base + lane;
        const bool valid = key <= pos;
        long long offset = 0;               // of the key's value
        float score = -INFINITY;
        if (valid) {
            const int page = table[key / page_tokens];
            if (page < 0) {
                atomicExch(error_flag, 2);
            } else {
                const long long place = (long long)kvh * page_tokens + (key % page_tokens);
                offset = (long long)page * value_page_stride + place * value_dim;
                const A* kv = k_cache + (long long)page * page_stride + place * head_dim;
                float s = 0.0f;
                for (int i = 0; i < head_dim; ++i) s += qs[i] * to_float(kv[i]);
                // a learned number per (head, distance back to the key), added to the scaled score as it is
                if (distance_bias) s += distance_bias[(size_t)h * (distance_last + 1) + min(pos - key, distance_last)];
                score = s;
            }
        }
        const float block_max = warp_max(score);
        const float new_max = fmaxf(running_max, block_max);
        if (new_max == -INFINITY) continue;          // nothing readable in this block of keys
        const float correction = expf(running_max - new_max);   // exp(-inf) = 0 on the first block
        const float p = score == -INFINITY ? 0.0f : expf(score - new_max);
        denom = denom * correction + warp_sum(p);
#pragma unroll
        for (int r = 0; r < kAccRegs; ++r) acc[r] *= correction;
        running_max = new_max;
        const int count = min(32, pos - base + 1);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, offset, j);
            const A* vv = v_cache + oj;
#pragma unroll
            for (int r = 0; r < kAccRegs; ++r) {
                const int i = lane + 32 * r;
                if (i < value_dim) acc[r] += pj * to_float(vv[i]);
            }
        }
    }
    const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    A* ov = out + ((size_t)t * q_heads + h) * value_dim;
#pragma unroll
    for (int r = 0; r < kAccRegs; ++r) {
        const int i = lane + 32 * r;
        if (i < value_dim) ov[i] = from_float<A>(acc[r] * inv);
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

// q: [tokens, q_row_stride] with head h at columns h*head_dim; out: [tokens, q_heads*value_dim]. value_dim 0: as wide
// as the keys. chunk > 0: a query reads the keys of its own chunk of that many positions (and no window).
// distance_bias: float32 [q_heads, distance_last + 1] or null; entry [h, min(n, distance_last)] is added to the scaled
// score of head h for a key n positions back.
CELEG_API int celeg_attention_generic(const void* q, int q_row_stride, void* out, const void* k_cache,
                                      const void* v_cache, long long page_stride, long long value_page_stride,
                                      int value_dim, int chunk, const int* positions,
                                      const int* token_span, const int* block_table, int table_stride,
                                      int tokens, int q_heads, int kv_heads, int head_dim, int page_tokens,
                                      int window, float scale, const float* sinks, const float* distance_bias,
                                      int distance_last, int* error_flag, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && page_tokens > 0,
                  "attention: invalid sizes tokens=%d q_heads=%d kv_heads=%d head_dim=%d page_tokens=%d", tokens,
                  q_heads, kv_heads, head_dim, page_tokens);
    CELEG_REQUIRE(q_heads % kv_heads == 0, "attention: %d query heads are not a multiple of %d kv heads", q_heads,
                  kv_heads);
    if (value_dim <= 0) {
        value_dim = head_dim;
        value_page_stride = page_stride;
    }
    CELEG_REQUIRE(value_dim <= 32 * kAccRegs, "attention: a value size of %d exceeds %d", value_dim, 32 * kAccRegs);
    CELEG_REQUIRE(chunk >= 0 && (chunk == 0 || window == 0), "attention: a chunk of %d beside a window of %d", chunk, window);
    if (tokens == 0) return 0;
    const int warps = 4;
    const long long units = (long long)tokens * q_heads;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    if (act_dtype == kFloat32)
        attention_generic_kernel<float><<<blocks, warps * 32, smem, stream>>>(
            (const float*)q, q_row_stride, (float*)out, (const float*)k_cache, (const float*)v_cache, page_stride,
            value_page_stride, positions, token_span, block_table, table_stride, tokens, q_heads, kv_heads, head_dim,
            value_dim, page_tokens, window, chunk, scale, sinks, distance_bias, distance_last, error_flag);
    else if (act_dtype == kBFloat16)
        attention_generic_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
            (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
            (const __nv_bfloat16*)v_cache, page_stride, value_page_stride, positions, token_span, block_table,
            table_stride, tokens, q_heads, kv_heads, head_dim, value_dim, page_tokens, window, chunk, scale, sinks,
            distance_bias, distance_last, error_flag);
    else
        CELEG_REQUIRE(false, "attention: unknown dtype code %d", act_dtype);
    return check_launch("attention_generic");
}

namespace celeg_b200 {

struct BiasStoreArgs {
    const float* proj; int proj_stride;       // rows [q heads | k heads | v heads] as projected, float32
    const float* bias;                        // as wide as a row's three parts together, or null
    void* q_out; int q_stride;                // queries in the activation type, head h at h * key_store
    const int* positions; const int* token_span; const int* block_table; int table_stride;
    void* k_cache; void* v_cache; long long page_stride, value_page_stride;
    int q_heads, kv_heads, head_dim, value_dim;    // sizes as projected
    int key_store, value_store;                    // sizes as stored (>= the projected ones; the rest is zero)
    int page_tokens;
    int* error_flag;
};

// The bias is added to the float32 sums and the result is rounded once: q goes to its buffer, k and v to the token's
// place in the paged cache. A stored head may be wider than the projected one (keys and values brought to one size
// for kernels that want them alike): the tail is written as zeros, which change no score and no result.
template <typename A>
__global__ void bias_store_kv_kernel(const BiasStoreArgs p) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int q_width = p.q_heads * p.head_dim, k_width = p.kv_heads * p.head_dim;
    const int q_store = p.q_heads * p.key_store, k_store = p.kv_heads * p.key_store, v_store = p.kv_heads * p.value_store;
    const int pos = p.positions[t];
    const int page = p.block_table[(size_t)p.token_span[t] * p.table_stride + pos / p.page_tokens];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(p.error_flag, 2);
    }
    const float* row = p.proj + (size_t)t * p.proj_stride;
    A* q_row = static_cast<A*>(p.q_out) + (size_t)t * p.q_stride;
    A* k_cache = static_cast<A*>(p.k_cache);
    A* v_cache = static_cast<A*>(p.v_cache);
    const long long in_page = pos % p.page_tokens;
    for (int i = threadIdx.x; i < q_store + k_store + v_store; i += blockDim.x) {
        if (i < q_store) {
            const int head = i / p.key_store, e = i % p.key_store;
            const int src = head * p.head_dim + e;
            q_row[i] = from_float<A>(e < p.head_dim ? row[src] + (p.bias ? p.bias[src] : 0.0f) : 0.0f);
        } else if (page >= 0) {
            if (i < q_store + k_store) {
                const int j = i - q_store, head = j / p.key_store, e = j % p.key_store;
                const int src = q_width + head * p.head_dim + e;
                k_cache[(long long)page * p.page_stride + ((long long)head * p.page_tokens + in_page) * p.key_store + e] =
                    from_float<A>(e < p.head_dim ? row[src] + (p.bias ? p.bias[src] : 0.0f) : 0.0f);
            } else {
                const int j = i - q_store - k_store, head = j / p.value_store, e = j % p.value_store;
                const int src = q_width + k_width + head * p.value_dim + e;
                v_cache[(long long)page * p.value_page_stride +
                        ((long long)head * p.page_tokens + in_page) * p.value_store + e] =
                    from_float<A>(e < p.value_dim ? row[src] + (p.bias ? p.bias[src] : 0.0f) : 0.0f);
            }
        }
    }
}

}  // namespace celeg_b200

// proj: float32 [tokens, proj_stride] rows [q | k | v] with heads of head_dim (q, k) and value_dim (v); q_out:
// [tokens, q_stride] in the activation type with heads of key_store; the caches hold heads of key_store and
// value_store.
CELEG_API int celeg_bias_store_kv(const float* proj, int proj_stride, const float* bias, void* q_out, int q_stride,
                                  const int* positions, const int* token_span, const int* block_table, int table_stride,
                                  void* k_cache, void* v_cache, long long page_stride, long long value_page_stride,
                                  int tokens, int q_heads, int kv_heads, int head_dim, int value_dim, int key_store,
                                  int value_store, int page_tokens, int* error_flag, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && value_dim > 0 && page_tokens > 0 &&
                  key_store >= head_dim && value_store >= value_dim && q_stride >= q_heads * key_store &&
                  proj_stride >= q_heads * head_dim + kv_heads * (head_dim + value_dim),
                  "bias_store_kv: invalid sizes tokens=%d q_heads=%d kv_heads=%d head_dim=%d value_dim=%d stored %d / %d "
                  "strides %d / %d", tokens, q_heads, kv_heads, head_dim, value_dim, key_store, value_store, proj_stride,
                  q_stride);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "bias_store_kv: unknown dtype code %d", act_dtype);
    if (tokens == 0) return 0;
    const BiasStoreArgs args = {proj, proj_stride, bias, q_out, q_stride, positions, token_span, block_table, table_stride,
                                k_cache, v_cache, page_stride, value_page_stride, q_heads, kv_heads, head_dim, value_dim,
                                key_store, value_store, page_tokens, error_flag};
    if (act_dtype == kFloat32)
        launch_chained(bias_store_kv_kernel<float>, tokens, 256, 0, stream, args);
    else
        launch_chained(bias_store_kv_kernel<__nv_bfloat16>, tokens, 256, 0, stream, args);
    return check_launch("bias_store_kv");
}
