// A gated linear recurrent unit over channels (De et al., "Griffin: Mixing Gated Linear Recurrences with Local
// Attention for Efficient Language Models", 2024: the real-gated linear recurrent unit of its recurrent block).
//
// Two branches of `width` channels come out of one projection [y | x] (float32 rows): the gate branch
// y' = gelu_tanh(y + b_y), and u = conv(x + b_x) + b_c, a causal depthwise convolution whose last tap meets the
// token itself and whose inputs before the start of a sequence are zero. The channels are cut into `blocks` equal
// parts; in part b the recurrence gate r = sigmoid(A_b u_b + a_b) and the input gate i = sigmoid(I_b u_b + i_b) are
// products with square matrices of the part's size. Per channel
//     a = exp(-c r softplus(lam)),    S <- a S + sqrt(1 - a^2) i u,    out = S y'
// with S float32 in the request's slot (zero for a new request, no special case for its first token), beside the
// last taps - 1 inputs x + b_x of the convolution. Everything here is float32 on both precision paths; `out` is
// written in the activation type for the projection that follows.
//
// Prompt portions: four launches (branches and convolution; the carried inputs; the gates' products, a batched
// FFMA product over the parts; decays and inputs element by element; the scan, a thread per channel walking its
// span over tiles that other warps stage in shared memory, so that the chain per token is one multiply-add). Steps in which every
// request brings one token: one launch, a block per (request, part).
#include "common.cuh"

namespace celeg_b200 {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// a and the input's factor sqrt(1 - a^2) from the recurrence gate r: log a = -c r softplus(lam); 1 - a^2 by expm1,
// which keeps its digits when a is close to 1
__device__ __forceinline__ void lru_decay(float r, float soft_lam, float c, float* a, float* in_scale) {
    const float log_a = -c * r * soft_lam;
    *a = expf(log_a);
    *in_scale = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.0f));
}

struct LruPrepareArgs {
    const float* proj; int stride;            // rows [y | x], `width` each
    const float* bias;                        // [2 * width]: b_y | b_x (null: none)
    const float* taps;                        // [width, n_taps]
    const float* conv_bias;                   // [width] (null: none)
    const float* carried;                     // inside slot 0: [n_taps - 1, width], oldest first, x + b_x
    long long slot_stride;
    const int* token_span; const int* span_begin; const int* span_slot;
    float* y_out; float* u_out;               // [tokens, width]
    int tokens, width, n_taps;
};

// One block a token: y' and u of every channel.
__global__ void lru_prepare_kernel(const LruPrepareArgs p) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int span = p.token_span[t];
    const int begin = p.span_begin[span];
    const float* carried = p.carried + (long long)p.span_slot[span] * p.slot_stride;
    const int rel = t - begin, width = p.width, n = p.n_taps;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float by = p.bias ? p.bias[c] : 0.0f, bx = p.bias ? p.bias[width + c] : 0.0f;
        p.y_out[(size_t)t * width + c] = activate(p.proj[(size_t)t * p.stride + c] + by, kGeluTanh);
        float sum = p.conv_bias ? p.conv_bias[c] : 0.0f;
        for (int j = 0; j < n; ++j) {
            const int s = rel - (n - 1) + j;
            const float x = s >= 0 ? p.proj[(size_t)(begin + s) * p.stride + width + c] + bx
                                   : carried[(size_t)(n - 1 + s) * width + c];
            sum = fmaf(p.taps[(size_t)c * n + j], x, sum);
        }
        p.u_out[(size_t)t * width + c] = sum;
    }
}

// The carried inputs after a step: the last n_taps - 1 inputs x + b_x of each request's sequence. One thread per
// (span, channel) reads everything it needs before it writes, so the update is in place.
__global__ void lru_carry_kernel(const float* proj, int stride, const float* bias, float* carried,
                                 long long slot_stride, const int* span_begin, const int* span_slot, int spans,
                                 int width, int n_taps) {
    chain_release();
    chain_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= spans * width) return;
    const int span = i / width, c = i % width;
    const int begin = span_begin[span], len = span_begin[span + 1] - begin;
    if (len <= 0) return;
    float* mine = carried + (long long)span_slot[span] * slot_stride;
    const float bx = bias ? bias[width + c] : 0.0f;
    float keep[15];
#pragma unroll
    for (int r = 0; r < 15; ++r) {
        if (r < n_taps - 1) {
            const int s = len - (n_taps - 1) + r;
            keep[r] = s >= 0 ? proj[(size_t)(begin + s) * stride + width + c] + bx
                             : mine[(size_t)(n_taps - 1 + s) * width + c];
        }
    }
#pragma unroll
    for (int r = 0; r < 15; ++r)
        if (r < n_taps - 1) mine[(size_t)r * width + c] = keep[r];
}

// Batched FFMA product over the parts: y[:, z * n + j] = sum_i x[:, (z % x_parts) * k + i] w[z][j][i], float32,
// ascending i, one thread an output element's whole sum (so a row does not depend on what else is in the batch).
constexpr int kBdTile = 64, kBdTileK = 16;
__global__ void __launch_bounds__(256) block_diagonal_kernel(const float* __restrict__ x, int ldx, int x_parts,
                                                             const float* __restrict__ w, float* __restrict__ y,
                                                             int ldy, int m, int n, int k) {
    __shared__ float xs[kBdTileK][kBdTile + 4];
    __shared__ float ws[kBdTileK][kBdTile + 4];
    chain_release();
    chain_wait();
    const int z = blockIdx.z;
    x += (size_t)(z % x_parts) * k;
    w += (size_t)z * n * k;
    y += (size_t)z * n;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int row0 = blockIdx.y * kBdTile, col0 = blockIdx.x * kBdTile;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < k; k0 += kBdTileK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gr = row0 + r, gc = col0 + r, gk = k0 + kk;
            xs[kk][r] = (gr < m && gk < k) ? x[(size_t)gr * ldx + gk] : 0.0f;
            ws[kk][r] = (gc < n && gk < k) ? w[(size_t)gc * k + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBdTileK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc < n) y[(size_t)gr * ldy + gc] = acc[i][j];
        }
    }
}

// Element by element: the gates' sums [tokens, 2 * width] (recurrence gate | input gate) become the decay a and the
// input b = sqrt(1 - a^2) i u, in place.
__global__ void lru_gates_kernel(float* gates, const float* u, const float* gate_bias, const float* lam, float c,
                                 long long total, int width) {
    chain_release();
    chain_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const long long t = idx / width;
        const int ch = (int)(idx % width);
        float* row = gates + t * 2 * width;
        const float r = sigmoid_f(row[ch] + (gate_bias ? gate_bias[ch] : 0.0f));
        const float i = sigmoid_f(row[width + ch] + (gate_bias ? gate_bias[width + ch] : 0.0f));
        float a, in_scale;
        lru_decay(r, softplus_f(lam[ch]), c, &a, &in_scale);
        row[ch] = a;
        row[width + ch] = in_scale * i * u[idx];
    }
}

__device__ __forceinline__ void lru_cp_async_4(void* smem, const void* global) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(global));
}
__device__ __forceinline__ void lru_cp_async_16(void* smem, const void* global) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(global));
}

// The scan: S <- a S + b per channel along a span, out = S y'. A block takes kLruChannels channels of one span; the
// tokens' a, b and y' arrive in tiles of kLruTile tokens through a ring of kLruStages stages (cp.async), so that the
// only thing a token waits for is the multiply-add of the token before it.
// One warp walks the chain of its 32 channels; three more warps of the block do nothing but copy (one the decays, one
// the inputs, one the y branch), so that the walking warp issues little besides the tile's loads from shared memory,
// its sixteen multiply-adds and its stores. Eight stages: seven tiles are under way while one is walked.
constexpr int kLruChannels = 32, kLruTile = 16, kLruStages = 8, kLruScanThreads = 128;
constexpr size_t kLruScanSmem = 3ull * kLruStages * kLruTile * kLruChannels * sizeof(float);
template <typename A>
__global__ void __launch_bounds__(kLruScanThreads) lru_scan_kernel(const float* __restrict__ gates,
                                                                   const float* __restrict__ y, A* __restrict__ out,
                                                                   float* state, long long slot_stride,
                                                                   const int* span_begin, const int* span_slot, int width,
                                                                   int vector_copies) {
    extern __shared__ __align__(16) float lru_scan_smem[];
    typedef float (*Ring)[kLruTile][kLruChannels];
    Ring a_s = reinterpret_cast<Ring>(lru_scan_smem);
    Ring b_s = a_s + kLruStages;
    Ring y_s = b_s + kLruStages;
    chain_release();
    chain_wait();
    const int span = blockIdx.y, c0 = blockIdx.x * kLruChannels;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t_begin = span_begin[span], t_end = span_begin[span + 1];
    if (t_end <= t_begin) return;
    const int c = c0 + lane;
    const bool walker = warp == 0, live = c < width;
    const int channels = min(kLruChannels, width - c0);
    float* cell = state + (long long)span_slot[span] * slot_stride + c;
    float s = walker && live ? *cell : 0.0f;
    // what a copying warp copies: rows of `ld` floats from `src` into `ring`
    const float* src = warp == 3 ? y + c0 : gates + (warp == 2 ? width : 0) + c0;
    const size_t ld = warp == 3 ? (size_t)width : 2 * (size_t)width;
    Ring ring = warp == 3 ? y_s : (warp == 2 ? b_s : a_s);
    auto issue = [&](int t0, int stage) {
        const int count = min(kLruTile, t_end - t0);
        if (count > 0) {
            if (vector_copies && channels == kLruChannels) {          // eight copies of 16 bytes a row, four a lane
#pragma unroll
                for (int i = lane; i < kLruTile * 8; i += 32) {
                    const int tt = i >> 3, e = (i & 7) << 2;
                    if (tt < count) lru_cp_async_16(&ring[stage][tt][e], src + (size_t)(t0 + tt) * ld + e);
                }
            } else if (vector_copies) {
                const int quads = channels >> 2;           // (width % 4 == 0, so channels % 4 == 0)
                for (int i = lane; i < count * quads; i += 32) {
                    const int tt = i / quads, e = (i - tt * quads) << 2;
                    lru_cp_async_16(&ring[stage][tt][e], src + (size_t)(t0 + tt) * ld + e);
                }
            } else {
                for (int i = lane; i < count * channels; i += 32) {
                    const int tt = i / channels, e = i - tt * channels;
                    lru_cp_async_4(&ring[stage][tt][e], src + (size_t)(t0 + tt) * ld + e);
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");       // (an empty group keeps the count of groups even)
    };
    if (!walker) {
#pragma unroll
        for (int ahead = 0; ahead < kLruStages - 1; ++ahead) issue(t_begin + ahead * kLruTile, ahead);
    }
    int stage = 0;
    for (int t0 = t_begin; t0 < t_end; t0 += kLruTile) {
        if (!walker) asm volatile("cp.async.wait_group %0;\n" ::"n"(kLruStages - 2) : "memory");
        // one barrier a tile: behind it this tile's copies have landed, and the walking warp is done with the tile
        // before, whose stage the copying warps fill next while this tile is walked
        __syncthreads();
        if (!walker) issue(t0 + (kLruStages - 1) * kLruTile, (stage + kLruStages - 1) % kLruStages);
        const int count = min(kLruTile, t_end - t0);
        if (walker && live) {
            A* dst = out + (size_t)t0 * width + c;
            if (count == kLruTile) {
                float av[kLruTile], bv[kLruTile], yv[kLruTile];
#pragma unroll
                for (int tt = 0; tt < kLruTile; ++tt) {
                    av[tt] = a_s[stage][tt][lane];
                    bv[tt] = b_s[stage][tt][lane];
                    yv[tt] = y_s[stage][tt][lane];
                }
#pragma unroll
                for (int tt = 0; tt < kLruTile; ++tt) {
                    s = fmaf(av[tt], s, bv[tt]);
                    dst[(size_t)tt * width] = from_float<A>(s * yv[tt]);
                }
            } else {
                for (int tt = 0; tt < count; ++tt) {
                    s = fmaf(a_s[stage][tt][lane], s, b_s[stage][tt][lane]);
                    dst[(size_t)tt * width] = from_float<A>(s * y_s[stage][tt][lane]);
                }
            }
        }
        stage = (stage + 1) % kLruStages;
    }
    if (walker && live) *cell = s;
}

// Decoding: every request brings one token. A block takes one part of one request's channels and does everything
// between the two projections for them: branches, convolution over the carried inputs (which it moves on), both
// gates' products (a warp an output channel, lanes over the part's inputs), decay, state and output.
struct LruDecodeArgs {
    const float* proj; int stride;
    const float* bias; const float* taps; const float* conv_bias;
    float* carried; float* state; long long slot_stride;
    const int* span_slot;
    const float* gate_w;                      // [2, blocks, part, part]
    const float* gate_bias;                   // [2 * width] (null: none)
    const float* lam; float c;
    void* out;                                // [tokens, width], activation type
    int width, n_taps, blocks;
};

template <typename A>
__global__ void __launch_bounds__(256) lru_decode_kernel(const LruDecodeArgs p) {
    extern __shared__ float lru_smem[];       // u of the part [part] | gate sums [2 * part]
    chain_release();
    chain_wait();
    const int part_index = blockIdx.x, t = blockIdx.y;
    const int width = p.width, n = p.n_taps, part = width / p.blocks;
    const int first = part_index * part;
    float* u_s = lru_smem;
    float* g_s = u_s + part;
    const float* row = p.proj + (size_t)t * p.stride;
    const long long slot_at = (long long)p.span_slot[t] * p.slot_stride;
    float* carried = p.carried + slot_at;
    for (int e = threadIdx.x; e < part; e += blockDim.x) {
        const int ch = first + e;
        const float x = row[width + ch] + (p.bias ? p.bias[width + ch] : 0.0f);
        float sum = p.conv_bias ? p.conv_bias[ch] : 0.0f;
        float older[15];
#pragma unroll
        for (int j = 0; j < 15; ++j)
            if (j < n - 1) older[j] = carried[(size_t)j * width + ch];
#pragma unroll
        for (int j = 0; j < 15; ++j)
            if (j < n - 1) sum = fmaf(p.taps[(size_t)ch * n + j], older[j], sum);
        sum = fmaf(p.taps[(size_t)ch * n + n - 1], x, sum);
        u_s[e] = sum;
        // the carried inputs move on by one: only this thread touches this channel's
#pragma unroll
        for (int j = 0; j < 15; ++j)
            if (j < n - 1) carried[(size_t)j * width + ch] = j + 1 < n - 1 ? older[j + 1] : x;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    // eight outputs a round, so that eight rows of the matrices are under way at once (each output's sum as before:
    // a lane its strided inputs in ascending order, then the warp's sum)
    constexpr int kOutputs = 8;
    for (int o0 = warp * kOutputs; o0 < 2 * part; o0 += warps * kOutputs) {
        const float* w[kOutputs];
        float sums[kOutputs];
#pragma unroll
        for (int q = 0; q < kOutputs; ++q) {
            const int o = min(o0 + q, 2 * part - 1);
            const int gate = o / part, j = o % part;
            w[q] = p.gate_w + (((size_t)gate * p.blocks + part_index) * part + j) * part;
            sums[q] = 0.0f;
        }
        for (int i = lane; i < part; i += 32) {
            const float uv = u_s[i];
#pragma unroll
            for (int q = 0; q < kOutputs; ++q) sums[q] = fmaf(w[q][i], uv, sums[q]);
        }
#pragma unroll
        for (int q = 0; q < kOutputs; ++q) {
            const float sum = warp_sum(sums[q]);
            if (lane == 0 && o0 + q < 2 * part) g_s[o0 + q] = sum;
        }
    }
    __syncthreads();
    A* dst = static_cast<A*>(p.out) + (size_t)t * width;
    float* state = p.state + slot_at;
    for (int e = threadIdx.x; e < part; e += blockDim.x) {
        const int ch = first + e;
        const float r = sigmoid_f(g_s[e] + (p.gate_bias ? p.gate_bias[ch] : 0.0f));
        const float i = sigmoid_f(g_s[part + e] + (p.gate_bias ? p.gate_bias[width + ch] : 0.0f));
        float a, in_scale;
        lru_decay(r, softplus_f(p.lam[ch]), p.c, &a, &in_scale);
        const float s = fmaf(a, state[ch], in_scale * i * u_s[e]);
        state[ch] = s;
        const float yv = activate(row[ch] + (p.bias ? p.bias[ch] : 0.0f), kGeluTanh);
        dst[ch] = from_float<A>(s * yv);
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

// Branches and convolution of a step's tokens, then the carried inputs moved on. proj: float32 [tokens, stride] rows
// [y | x]; bias [2 * width] or null; taps [width, n_taps]; conv_bias [width] or null; carried: this part's carried
// inputs inside slot 0. y_out, u_out: float32 [tokens, width].
CELEG_API int celeg_lru_prepare(const float* proj, int stride, const float* bias, const float* taps,
                                const float* conv_bias, float* carried, long long slot_stride, const int* token_span,
                                const int* span_begin, const int* span_slot, float* y_out, float* u_out, int tokens,
                                int spans, int width, int n_taps, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && spans >= 0 && width > 0 && n_taps >= 1 && n_taps <= 16 && stride >= 2 * width,
                  "lru_prepare: invalid sizes tokens=%d width=%d taps=%d stride=%d", tokens, width, n_taps, stride);
    if (tokens == 0) return 0;
    const LruPrepareArgs args = {proj, stride, bias, taps, conv_bias, carried, slot_stride, token_span, span_begin,
                                 span_slot, y_out, u_out, tokens, width, n_taps};
    launch_chained(lru_prepare_kernel, tokens, 256, 0, stream, args);
    int status = check_launch("lru_prepare");
    if (status != 0 || n_taps == 1) return status;
    const long long units = (long long)spans * width;
    launch_chained(lru_carry_kernel, (unsigned)((units + 127) / 128), 128, 0, stream, proj, stride, bias, carried,
                   slot_stride, span_begin, span_slot, spans, width, n_taps);
    return check_launch("lru_carry");
}

// y[:, z * n : (z + 1) * n] = x[:, (z % x_parts) * k : ...] w[z]^T for z < batches; float32 throughout.
CELEG_API int celeg_block_diagonal_product(const float* x, int ldx, int x_parts, const float* w, float* y, int ldy,
                                           int m, int n, int k, int batches, cudaStream_t stream) {
    CELEG_REQUIRE(m >= 0 && n > 0 && k > 0 && batches > 0 && x_parts > 0 && ldx >= x_parts * k && ldy >= batches * n,
                  "block_diagonal_product: invalid sizes m=%d n=%d k=%d batches=%d parts=%d ldx=%d ldy=%d", m, n, k,
                  batches, x_parts, ldx, ldy);
    if (m == 0) return 0;
    dim3 grid((n + kBdTile - 1) / kBdTile, (m + kBdTile - 1) / kBdTile, batches);
    CELEG_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "block_diagonal_product: %d rows or %d batches exceed one launch", m,
                  batches);
    launch_chained(block_diagonal_kernel, grid, 256, 0, stream, x, ldx, x_parts, w, y, ldy, m, n, k);
    return check_launch("block_diagonal_product");
}

// gates: float32 [tokens, 2 * width], the gates' sums, rewritten as (a | b); then the scan over the spans with the
// state inside the slots, out [tokens, width] = S y' in the activation type.
CELEG_API int celeg_lru_scan(float* gates, const float* u, const float* gate_bias, const float* lam, float c,
                             const float* y, void* out, float* state, long long slot_stride, const int* span_begin,
                             const int* span_slot, int tokens, int spans, int width, int act_dtype,
                             cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && spans >= 0 && width > 0 && c > 0.0f, "lru_scan: invalid sizes tokens=%d spans=%d width=%d",
                  tokens, spans, width);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "lru_scan: unknown dtype code %d", act_dtype);
    CELEG_REQUIRE(spans <= 65535, "lru_scan: %d spans exceed one launch", spans);
    if (tokens == 0 || spans == 0) return 0;
    const long long total = (long long)tokens * width;
    const long long wanted = (total + 255) / 256;
    launch_chained(lru_gates_kernel, (unsigned)(wanted < 148LL * 16 ? wanted : 148LL * 16), 256, 0, stream, gates, u,
                   gate_bias, lam, c, total, width);
    int status = check_launch("lru_gates");
    if (status != 0) return status;
    const int vector_copies = width % 4 == 0 && (((size_t)gates | (size_t)y) & 15) == 0;
    dim3 grid((width + kLruChannels - 1) / kLruChannels, spans);
    static bool sized = false;
    if (!sized) {
        if (cudaFuncSetAttribute(lru_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLruScanSmem) != cudaSuccess ||
            cudaFuncSetAttribute(lru_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLruScanSmem) != cudaSuccess)
            CELEG_REQUIRE(false, "lru_scan: %zu bytes of shared memory were refused", kLruScanSmem);
        sized = true;
    }
    if (act_dtype == kFloat32)
        launch_chained(lru_scan_kernel<float>, grid, kLruScanThreads, kLruScanSmem, stream, (const float*)gates, y, (float*)out, state,
                       slot_stride, span_begin, span_slot, width, vector_copies);
    else
        launch_chained(lru_scan_kernel<__nv_bfloat16>, grid, kLruScanThreads, kLruScanSmem, stream, (const float*)gates, y,
                       (__nv_bfloat16*)out, state, slot_stride, span_begin, span_slot, width, vector_copies);
    return check_launch("lru_scan");
}

// One token per request (row i of proj is request i's token, its slot span_slot[i]): the whole unit in one launch.
CELEG_API int celeg_lru_decode(const float* proj, int stride, const float* bias, const float* taps,
                               const float* conv_bias, float* carried, float* state, long long slot_stride,
                               const int* span_slot, const float* gate_w, const float* gate_bias, const float* lam,
                               float c, void* out, int tokens, int width, int n_taps, int blocks, int act_dtype,
                               cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && tokens <= 65535 && width > 0 && blocks > 0 && width % blocks == 0 && n_taps >= 1 &&
                  n_taps <= 16 && stride >= 2 * width && c > 0.0f,
                  "lru_decode: invalid sizes tokens=%d width=%d blocks=%d taps=%d stride=%d", tokens, width, blocks, n_taps,
                  stride);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "lru_decode: unknown dtype code %d", act_dtype);
    const int part = width / blocks;
    const size_t smem = (size_t)3 * part * sizeof(float);
    CELEG_REQUIRE(smem <= 48 * 1024, "lru_decode: a part of %d channels exceeds a block's shared memory", part);
    if (tokens == 0) return 0;
    const LruDecodeArgs args = {proj, stride, bias, taps, conv_bias, carried, state, slot_stride, span_slot, gate_w,
                                gate_bias, lam, c, out, width, n_taps, blocks};
    dim3 grid(blocks, tokens);
    if (act_dtype == kFloat32)
        launch_chained(lru_decode_kernel<float>, grid, 256, smem, stream, args);
    else
        launch_chained(lru_decode_kernel<__nv_bfloat16>, grid, 256, smem, stream, args);
    return check_launch("lru_decode");
}
