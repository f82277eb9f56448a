// Fused residual add + layer norm (mean-centred) with an optional row gather, and two small row kernels that
// mixers use between their products.
//
//   x = residual[r] (+ delta[r]);  residual[r] = x (if asked);
//   out[i] = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w (+ b)
//
// with r = rows[i] when a row list is given, else r = i. Two passes over values a thread keeps in registers: the
// mean first, then the mean of the squared deviations from it (not E[x^2] - mean^2, which loses digits when the
// mean is large beside the spread). Sums, the reciprocal root and the affine part are float32; the result is
// rounded once to the activation type.
//
//   rmsnorm_strided   y[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w over `width` columns of rows that lie `stride`
//                     elements apart (a slice of a fused projection's result)
//   sigmoid_gate      values[t, c] *= sigmoid(gate[t, c]) in place, gate float32 or of the activation type
#include "common.cuh"

namespace celeg_b200 {

template <typename A, int kPerThread>
__global__ void add_layernorm_kernel(float* residual, const A* delta, const float* __restrict__ weight,
                                     const float* __restrict__ bias, A* out, const int* rows, int width, float eps,
                                     int write_residual) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * width;
    const A* del = delta ? delta + (size_t)r * width : nullptr;
    float x[kPerThread];
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int c = threadIdx.x + u * blockDim.x;
        float v = 0.0f;
        if (c < width) {
            v = res[c];
            if (del) {
                v += to_float(del[c]);
                if (write_residual) res[c] = v;
            }
        }
        x[u] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)width;
    float squares = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int c = threadIdx.x + u * blockDim.x;
        const float dev = c < width ? x[u] - mean : 0.0f;
        x[u] = dev;
        squares += dev * dev;
    }
    const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
    A* dst = out + (size_t)i * width;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int c = threadIdx.x + u * blockDim.x;
        if (c < width) dst[c] = from_float<A>(x[u] * inv * weight[c] + (bias ? bias[c] : 0.0f));
    }
}

// Widths that are a multiple of 4 with 16-byte aligned rows: four elements a load, a thread's elements in registers
// between the passes (the stream is read once).
template <typename A, int kPerThread>
__global__ void add_layernorm_vec4_kernel(float* residual, const A* delta, const float* __restrict__ weight,
                                          const float* __restrict__ bias, A* out, const int* rows, int width, float eps,
                                          int write_residual) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float4* res = reinterpret_cast<float4*>(residual + (size_t)r * width);
    const int quads = width >> 2;
    float4 x[kPerThread];
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int q = threadIdx.x + u * blockDim.x;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (q < quads) {
            v = res[q];
            if (delta) {
                const A* d = delta + (size_t)r * width + 4 * q;
                if (sizeof(A) == 2) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(d);
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    v.x += lo.x; v.y += lo.y; v.z += hi.x; v.w += hi.y;
                } else {
                    const float4 dv = *reinterpret_cast<const float4*>(d);
                    v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
                }
                if (write_residual) res[q] = v;
            }
        }
        x[u] = v;
        sum += (v.x + v.y) + (v.z + v.w);
    }
    const float mean = block_sum(sum, scratch) / (float)width;
    float squares = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int q = threadIdx.x + u * blockDim.x;
        if (q < quads) {
            float4 v = x[u];
            v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
            x[u] = v;
            squares += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int q = threadIdx.x + u * blockDim.x;
        if (q < quads) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(weight) + q);
            const float4 b = bias ? __ldg(reinterpret_cast<const float4*>(bias) + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float4 v = x[u];
            const float4 y = make_float4(v.x * inv * w.x + b.x, v.y * inv * w.y + b.y, v.z * inv * w.z + b.z,
                                         v.w * inv * w.w + b.w);
            A* dst = out + (size_t)i * width + 4 * q;
            if (sizeof(A) == 2) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(y.z, y.w);
                uint2 raw;
                raw.x = *reinterpret_cast<const unsigned*>(&lo);
                raw.y = *reinterpret_cast<const unsigned*>(&hi);
                *reinterpret_cast<uint2*>(dst) = raw;
            } else {
                *reinterpret_cast<float4*>(dst) = y;
            }
        }
    }
}

// rows wider than a block's registers hold: three passes over memory
template <typename A>
__global__ void add_layernorm_wide_kernel(float* residual, const A* delta, const float* __restrict__ weight,
                                          const float* __restrict__ bias, A* out, const int* rows, int width, float eps,
                                          int write_residual) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * width;
    const A* del = delta ? delta + (size_t)r * width : nullptr;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) sum += res[c] + (del ? to_float(del[c]) : 0.0f);
    const float mean = block_sum(sum, scratch) / (float)width;
    float squares = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float dev = res[c] + (del ? to_float(del[c]) : 0.0f) - mean;
        squares += dev * dev;
    }
    const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
    A* dst = out + (size_t)i * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = res[c] + (del ? to_float(del[c]) : 0.0f);
        if (write_residual && del) res[c] = v;
        dst[c] = from_float<A>((v - mean) * inv * weight[c] + (bias ? bias[c] : 0.0f));
    }
}

template <typename A>
__global__ void rmsnorm_strided_kernel(const A* in, long long in_stride, const float* __restrict__ weight, A* out,
                                       long long out_stride, int width, float eps) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const A* src = in + (size_t)blockIdx.x * in_stride;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float x = to_float(src[c]);
        sum += x * x;
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)width + eps);
    A* dst = out + (size_t)blockIdx.x * out_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = from_float<A>(to_float(src[c]) * inv * weight[c]);
}

template <typename A, typename G>
__global__ void sigmoid_gate_kernel(A* values, long long stride, const G* gate, long long gate_stride, int tokens,
                                    int width) {
    chain_release();
    chain_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    const float g = 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + c])));
    A* cell = values + (size_t)t * stride + c;
    *cell = from_float<A>(to_float(*cell) * g);
}

// four neighbours a thread (rows whose widths and strides are multiples of four, 16-byte aligned gate rows)
template <typename A, typename G>
__global__ void sigmoid_gate_vec4_kernel(A* values, long long stride, const G* gate, long long gate_stride, int tokens,
                                         int width) {
    chain_release();
    chain_wait();
    const int quads = width >> 2;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * quads) return;
    const int t = (int)(i / quads), c = 4 * (int)(i % quads);
    A* cell = values + (size_t)t * stride + c;
    const G* g = gate + (size_t)t * gate_stride + c;
    float v[4], z[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        v[e] = to_float(cell[e]);
        z[e] = to_float(g[e]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) cell[e] = from_float<A>(v[e] / (1.0f + __expf(-z[e])));
}

template <typename A>
static void launch_layernorm(float* residual, const void* delta, const float* weight, const float* bias, void* out,
                             const int* rows, int n_rows, int width, float eps, int write_residual, cudaStream_t stream) {
    constexpr int kPerThread = 8;
    constexpr int kQuads = 4;
    const bool aligned = (((size_t)residual | (size_t)delta | (size_t)weight | (size_t)bias | (size_t)out) & 15) == 0;
    if (width % 4 == 0 && width <= 1024 * 4 * kQuads && aligned) {
        int threads = (width / 4 + kQuads - 1) / kQuads;
        threads = (threads + 31) / 32 * 32;
        if (threads < 64) threads = 64;
        launch_chained_class(kChainNorm, add_layernorm_vec4_kernel<A, kQuads>, n_rows, threads, 0, stream, residual,
                             (const A*)delta, weight, bias, (A*)out, rows, width, eps, write_residual);
    } else if (width <= 1024 * kPerThread) {
        int threads = (width + kPerThread - 1) / kPerThread;
        threads = (threads + 31) / 32 * 32;
        if (threads < 64) threads = 64;
        launch_chained_class(kChainNorm, add_layernorm_kernel<A, kPerThread>, n_rows, threads, 0, stream, residual,
                             (const A*)delta, weight, bias, (A*)out, rows, width, eps, write_residual);
    } else {
        launch_chained_class(kChainNorm, add_layernorm_wide_kernel<A>, n_rows, 1024, 0, stream, residual, (const A*)delta,
                             weight, bias, (A*)out, rows, width, eps, write_residual);
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_add_layernorm(float* residual, const void* delta, const float* weight, const float* bias, void* out,
                                  const int* rows, int n_rows, int width, float eps, int write_residual, int act_dtype,
                                  cudaStream_t stream) {
    CELEG_REQUIRE(n_rows >= 0 && width > 0 && eps > 0.0f, "add_layernorm: invalid sizes rows=%d width=%d eps=%g", n_rows,
                  width, eps);
    CELEG_REQUIRE(!(rows && write_residual), "add_layernorm: a gathered norm does not write the residual back");
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "add_layernorm: unknown dtype code %d", act_dtype);
    if (n_rows == 0) return 0;
    if (act_dtype == kFloat32)
        launch_layernorm<float>(residual, delta, weight, bias, out, rows, n_rows, width, eps, write_residual, stream);
    else
        launch_layernorm<__nv_bfloat16>(residual, delta, weight, bias, out, rows, n_rows, width, eps, write_residual,
                                        stream);
    return check_launch("add_layernorm");
}

CELEG_API int celeg_rmsnorm_strided(const void* in, long long in_stride, const float* weight, void* out,
                                    long long out_stride, int n_rows, int width, float eps, int act_dtype,
                                    cudaStream_t stream) {
    CELEG_REQUIRE(n_rows >= 0 && width > 0 && eps > 0.0f && in_stride >= width && out_stride >= width,
                  "rmsnorm_strided: invalid sizes rows=%d width=%d strides %lld / %lld eps=%g", n_rows, width, in_stride,
                  out_stride, eps);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "rmsnorm_strided: unknown dtype code %d", act_dtype);
    if (n_rows == 0) return 0;
    const int threads = width >= 2048 ? 512 : width >= 512 ? 256 : 128;
    if (act_dtype == kFloat32)
        launch_chained(rmsnorm_strided_kernel<float>, n_rows, threads, 0, stream, (const float*)in, in_stride, weight,
                       (float*)out, out_stride, width, eps);
    else
        launch_chained(rmsnorm_strided_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, (const __nv_bfloat16*)in,
                       in_stride, weight, (__nv_bfloat16*)out, out_stride, width, eps);
    return check_launch("rmsnorm_strided");
}

// gate_dtype: the type of `gate` (float32 sums of a product, or the activation type)
CELEG_API int celeg_sigmoid_gate(void* values, long long stride, const void* gate, long long gate_stride, int tokens,
                                 int width, int act_dtype, int gate_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && width > 0 && stride >= width && gate_stride >= width,
                  "sigmoid_gate: invalid sizes tokens=%d width=%d strides %lld / %lld", tokens, width, stride, gate_stride);
    CELEG_REQUIRE((act_dtype == kFloat32 || act_dtype == kBFloat16) && (gate_dtype == kFloat32 || gate_dtype == act_dtype),
                  "sigmoid_gate: dtype codes %d / %d", act_dtype, gate_dtype);
    if (tokens == 0) return 0;
    if (act_dtype == kBFloat16 && gate_dtype == kFloat32 && width % 4 == 0 && stride % 4 == 0 && gate_stride % 4 == 0) {
        const unsigned quad_blocks = (unsigned)(((long long)tokens * (width / 4) + 255) / 256);
        launch_chained(sigmoid_gate_vec4_kernel<__nv_bfloat16, float>, quad_blocks, 256, 0, stream, (__nv_bfloat16*)values,
                       stride, (const float*)gate, gate_stride, tokens, width);
        return check_launch("sigmoid_gate");
    }
    const unsigned blocks = (unsigned)(((long long)tokens * width + 255) / 256);
    if (act_dtype == kFloat32)
        launch_chained(sigmoid_gate_kernel<float, float>, blocks, 256, 0, stream, (float*)values, stride,
                       (const float*)gate, gate_stride, tokens, width);
    else if (gate_dtype == kFloat32)
        launch_chained(sigmoid_gate_kernel<__nv_bfloat16, float>, blocks, 256, 0, stream, (__nv_bfloat16*)values, stride,
                       (const float*)gate, gate_stride, tokens, width);
    else
        launch_chained(sigmoid_gate_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)values,
                       stride, (const __nv_bfloat16*)gate, gate_stride, tokens, width);
    return check_launch("sigmoid_gate");
}
