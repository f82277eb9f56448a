// Dynamic Tanh norm on the residual stream, and the element-wise pieces of blocks that use it.
//
//   x = residual[r] (+ delta_a[r]) (+ delta_b[r]);   residual[r] = x (if asked)
//   out_1[i] = tanh(alpha_1 x) w_1 + b_1             and, for a block whose mixer and feed-forward read the
//   out_2[i] = tanh(alpha_2 x) w_2 + b_2             same stream through a norm each, the second in the same pass
//
// with r = rows[i] when a row list is given (the rows whose logits are wanted), else r = i. The norm takes
// no mean and no variance, so there is no reduction: a thread a column of a row. Sum, tanh and
// the affine part are float32; the result is rounded once to the activation type.
//
// Also here: the stream joined with the embedding rows of the step's tokens (what a repeated run of layers
// is entered through), the exact and the tanh GELU, and the capped logits cap * tanh(x / cap).
#include "common.cuh"

namespace celeg_b200 {

struct DytArgs {
    float* residual;
    const void* delta_a;
    const void* delta_b;
    const int* rows;
    int n_rows, width, write_residual;
    const float* w1; const float* b1; float alpha1; void* out1;
    const float* w2; const float* b2; float alpha2; void* out2;
};

template <typename A>
__global__ void add_dyt_kernel(const DytArgs a) {
    chain_release();
    chain_wait();
    const int i = blockIdx.y;
    const int r = a.rows ? a.rows[i] : i;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.width) return;
    const size_t at = (size_t)r * a.width + c;
    float x = a.residual[at];
    if (a.delta_a) x += to_float(static_cast<const A*>(a.delta_a)[at]);
    if (a.delta_b) x += to_float(static_cast<const A*>(a.delta_b)[at]);
    if (a.write_residual && (a.delta_a || a.delta_b)) a.residual[at] = x;
    const size_t to = (size_t)i * a.width + c;
    if (a.out1) static_cast<A*>(a.out1)[to] = from_float<A>(tanhf(a.alpha1 * x) * a.w1[c] + a.b1[c]);
    if (a.out2) static_cast<A*>(a.out2)[to] = from_float<A>(tanhf(a.alpha2 * x) * a.w2[c] + a.b2[c]);
}

// joined[t] = [residual[t] (+ delta_a[t]) (+ delta_b[t]) | multiplier * table[token[t]]], in the activation type
template <typename A, typename W>
__global__ void join_stream_embedding_kernel(const float* residual, const A* delta_a, const A* delta_b,
                                             const W* __restrict__ table, const int* tokens, A* joined, int width,
                                             int vocab, float multiplier) {
    chain_release();
    chain_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const size_t at = (size_t)t * width + c;
    float x = residual[at];
    if (delta_a) x += to_float(delta_a[at]);
    if (delta_b) x += to_float(delta_b[at]);
    const int token = tokens[t];
    const bool valid = token >= 0 && token < vocab;          // the host refuses other ids before launch
    const float e = valid ? to_float(table[(size_t)token * width + c]) * multiplier : 0.0f;
    joined[(size_t)t * 2 * width + c] = from_float<A>(x);
    joined[(size_t)t * 2 * width + width + c] = from_float<A>(e);
}

template <typename A>
__global__ void activation_kernel(const A* in, A* out, long long count, int kind) {
    chain_release();
    chain_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = from_float<A>(activate(to_float(in[i]), kind));
}

// 16 bytes a thread: eight bfloat16 or four float32 (count a multiple of that, both pointers 16-byte aligned)
template <typename A>
__global__ void activation_vec_kernel(const uint4* in, uint4* out, long long vectors, int kind) {
    chain_release();
    chain_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= vectors) return;
    uint4 raw = in[i];
    if (sizeof(A) == 2) {
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 z = __bfloat1622float2(pairs[j]);
            pairs[j] = __floats2bfloat162_rn(activate(z.x, kind), activate(z.y, kind));
        }
    } else {
        float* z = reinterpret_cast<float*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) z[j] = activate(z[j], kind);
    }
    out[i] = raw;
}

__global__ void softcap_kernel(float* logits, long long count, float cap, float inv_cap) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) logits[i] = cap * tanhf(logits[i] * inv_cap);
}

}  // namespace celeg_b200

using namespace celeg_b200;

// Either output may be null (with its weights); delta_a / delta_b may be null. rows != null gathers and
// leaves the residual alone.
CELEG_API int celeg_add_dyt(float* residual, const void* delta_a, const void* delta_b, const int* rows, int n_rows,
                            int width, int write_residual, const float* w1, const float* b1, float alpha1, void* out1,
                            const float* w2, const float* b2, float alpha2, void* out2, int act_dtype,
                            cudaStream_t stream) {
    CELEG_REQUIRE(n_rows >= 0 && width > 0, "add_dyt: invalid sizes rows=%d width=%d", n_rows, width);
    CELEG_REQUIRE(!(rows && write_residual), "add_dyt: a gathered norm does not write the residual back");
    CELEG_REQUIRE((!out1 || (w1 && b1)) && (!out2 || (w2 && b2)), "add_dyt: an output needs its weight and bias");
    CELEG_REQUIRE(n_rows <= 65535 * 1, "add_dyt: %d rows exceed one launch", n_rows);
    if (n_rows == 0) return 0;
    const DytArgs args = {residual, delta_a, delta_b, rows, n_rows, width, write_residual,
                          w1, b1, alpha1, out1, w2, b2, alpha2, out2};
    const int threads = width >= 256 ? 256 : 128;
    dim3 grid((width + threads - 1) / threads, n_rows);
    if (act_dtype == kFloat32)
        launch_chained_class(kChainNorm, add_dyt_kernel<float>, grid, threads, 0, stream, args);
    else if (act_dtype == kBFloat16)
        launch_chained_class(kChainNorm, add_dyt_kernel<__nv_bfloat16>, grid, threads, 0, stream, args);
    else
        CELEG_REQUIRE(false, "add_dyt: unknown dtype code %d", act_dtype);
    return check_launch("add_dyt");
}

CELEG_API int celeg_join_stream_embedding(const float* residual, const void* delta_a, const void* delta_b,
                                          const void* table, const int* tokens, void* joined, int n_rows, int width,
                                          int vocab, float multiplier, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(n_rows >= 0 && width > 0 && vocab > 0, "join_stream_embedding: invalid sizes rows=%d width=%d vocab=%d",
                  n_rows, width, vocab);
    CELEG_REQUIRE(n_rows <= 65535, "join_stream_embedding: %d rows exceed one launch", n_rows);
    if (n_rows == 0) return 0;
    const int threads = width >= 256 ? 256 : 128;
    dim3 grid((width + threads - 1) / threads, n_rows);
    if (act_dtype == kFloat32)
        launch_chained(join_stream_embedding_kernel<float, float>, grid, threads, 0, stream, residual,
                       (const float*)delta_a, (const float*)delta_b, (const float*)table, tokens, (float*)joined,
                       width, vocab, multiplier);
    else if (act_dtype == kBFloat16)
        launch_chained(join_stream_embedding_kernel<__nv_bfloat16, __nv_bfloat16>, grid, threads, 0, stream, residual,
                       (const __nv_bfloat16*)delta_a, (const __nv_bfloat16*)delta_b, (const __nv_bfloat16*)table,
                       tokens, (__nv_bfloat16*)joined, width, vocab, multiplier);
    else
        CELEG_REQUIRE(false, "join_stream_embedding: unknown dtype code %d", act_dtype);
    return check_launch("join_stream_embedding");
}

// out = act(in), element by element (in place allowed): 0 the exact GELU, 1 the tanh GELU, 2 SiLU
namespace celeg_b200 {
// act() of the first `columns` columns of every row, in place; the rest of a row is left alone
template <typename A>
__global__ void activation_columns_kernel(A* x, long long stride, int columns, long long count, int kind) {
    chain_release();
    chain_wait();
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
        A* cell = x + (i / columns) * stride + (i % columns);
        *cell = from_float<A>(activate(to_float(*cell), kind));
    }
}
}  // namespace celeg_b200

CELEG_API int celeg_activation_columns(void* x, long long stride, int columns, int rows, int kind, int act_dtype,
                                       cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && columns > 0 && stride >= columns && kind >= 0 && kind <= 4,
                  "activation_columns: invalid sizes rows=%d columns=%d kind=%d", rows, columns, kind);
    if (rows == 0) return 0;
    const long long count = (long long)rows * columns;
    const long long wanted = (count + 255) / 256;
    const unsigned blocks = (unsigned)(wanted < 148LL * 16 ? wanted : 148LL * 16);
    if (act_dtype == kFloat32)
        launch_chained(activation_columns_kernel<float>, blocks, 256, 0, stream, (float*)x, stride, columns, count, kind);
    else if (act_dtype == kBFloat16)
        launch_chained(activation_columns_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)x, stride, columns,
                       count, kind);
    else
        CELEG_REQUIRE(false, "activation_columns: unknown dtype code %d", act_dtype);
    return check_launch("activation_columns");
}

CELEG_API int celeg_activation(const void* in, void* out, long long count, int kind, int act_dtype,
                               cudaStream_t stream) {
    CELEG_REQUIRE(count >= 0 && kind >= 0 && kind <= 4, "activation: invalid count %lld or kind %d", count, kind);
    if (count == 0) return 0;
    const int per_vector = act_dtype == kFloat32 ? 4 : 8;
    if ((act_dtype == kFloat32 || act_dtype == kBFloat16) && count % per_vector == 0 &&
        (((size_t)in | (size_t)out) & 15) == 0) {
        const long long vectors = count / per_vector;
        const unsigned vec_blocks = (unsigned)((vectors + 255) / 256);
        if (act_dtype == kFloat32)
            launch_chained(activation_vec_kernel<float>, vec_blocks, 256, 0, stream, (const uint4*)in, (uint4*)out,
                           vectors, kind);
        else
            launch_chained(activation_vec_kernel<__nv_bfloat16>, vec_blocks, 256, 0, stream, (const uint4*)in,
                           (uint4*)out, vectors, kind);
        return check_launch("activation");
    }
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (act_dtype == kFloat32)
        launch_chained(activation_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, count, kind);
    else if (act_dtype == kBFloat16)
        launch_chained(activation_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)in,
                       (__nv_bfloat16*)out, count, kind);
    else
        CELEG_REQUIRE(false, "activation: unknown dtype code %d", act_dtype);
    return check_launch("activation");
}

CELEG_API int celeg_softcap(float* logits, long long count, float cap, cudaStream_t stream) {
    CELEG_REQUIRE(count >= 0 && cap > 0.0f, "softcap: invalid count %lld or cap %g", count, cap);
    if (count == 0) return 0;
    softcap_kernel<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(logits, count, cap, 1.0f / cap);
    return check_launch("softcap");
}

namespace celeg_b200 {
// out = scale_a (a + bias_a) + scale_b b: the results of two mixers of the same input, side by side, as one output
// owed to the stream. a, b float32 [rows, width] (b null: no second term); bias_a [width] or null; float32
// arithmetic, rounded once.
template <typename A>
__global__ void scaled_sum_kernel(const float* a, const float* b, const float* bias_a, float scale_a, float scale_b,
                                  A* out, long long count, int width) {
    chain_release();
    chain_wait();
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
        const float left = a[i] + (bias_a ? bias_a[i % width] : 0.0f);
        out[i] = from_float<A>(b ? fmaf(scale_a, left, scale_b * b[i]) : scale_a * left);
    }
}
}  // namespace celeg_b200

CELEG_API int celeg_scaled_sum(const float* a, const float* b, const float* bias_a, float scale_a, float scale_b,
                               void* out, int rows, int width, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && width > 0, "scaled_sum: invalid sizes rows=%d width=%d", rows, width);
    if (rows == 0) return 0;
    const long long count = (long long)rows * width;
    const long long wanted = (count + 255) / 256;
    const unsigned blocks = (unsigned)(wanted < 148LL * 16 ? wanted : 148LL * 16);
    if (act_dtype == kFloat32)
        launch_chained(scaled_sum_kernel<float>, blocks, 256, 0, stream, a, b, bias_a, scale_a, scale_b, (float*)out, count,
                       width);
    else if (act_dtype == kBFloat16)
        launch_chained(scaled_sum_kernel<__nv_bfloat16>, blocks, 256, 0, stream, a, b, bias_a, scale_a, scale_b,
                       (__nv_bfloat16*)out, count, width);
    else
        CELEG_REQUIRE(false, "scaled_sum: unknown dtype code %d", act_dtype);
    return check_launch("scaled_sum");
}
