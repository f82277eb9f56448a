// Mixers whose cache is a matrix per head that every token rewrites: the mLSTM matrix memory, the gated
// delta rule and the retention (a fixed decay per head). State, gates and every sum are float32 on both
// precision paths.
//
// The recurrences, per head, with S [dim, vdim] (and for the mLSTM a normaliser n [dim] and a running
// maximum m that starts at 0):
//
//   mLSTM   m' = max(f + m, i);  a = exp(f + m - m'),  b = exp(i - m')
//           S' = a S + b k v^T;  n' = a n + b k;  o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
//   delta   S~ = g S;  u = beta (v - S~^T k);  S' = S~ + k u^T;  o = S'^T q
//   retention   S' = d S + k v^T;  o = S'^T q   with d a constant of the head (`gates` holds one per head, not per
//           token) and k the projected key times q_scale (dim^(-1/2)): the factor is applied to the value that is
//           written and to k.q, so S is the sum of scaled keys
//
// Column j of S depends on column j alone, so a launch is cut by (span, head, run of columns) and walks the
// span's tokens in order. A column lives in the registers of L lanes (L = 1 .. 32 by the key size, 8
// elements a lane); per token the lanes form S.k, S.q (and n.q) on the OLD state together, exchange them with
// shuffles once, and get the read-out from them without a second pass over the new state:
//   delta: o_j = g (S.q)_j + u_j (k.q)         mLSTM: (S'^T q)_j = a (S.q)_j + b v_j (k.q),  n'.q = a n.q + b k.q
// Keys, queries, values and gates of the next 16 tokens are copied to shared memory (cp.async) while the
// current 16 are worked on; the four warps of a block share them. A span of one token (decoding) is the same kernel: one state read, one write.
//
// Beside the scans: the gates of both mixers from their projections, the delta rule's short convolutions with
// their carried inputs, unit norms and decay, and the per-head norm with the output gate.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kScanRegs = 8;         // elements of a column a lane holds
constexpr int kScanWarps = 4;        // warps of a block: they share the staged keys and queries
constexpr int kScanThreads = kScanWarps * 32;
constexpr int kScanMaxDim = 256;

enum ScanMode : int { kScanDelta = 0, kScanMlstm = 1, kScanRetention = 2 };

struct ScanParams {
    const float* q; const float* k; const float* v;     // rows of the step's tokens; head h at h * dim (h * vdim)
    int q_stride, k_stride, v_stride;
    const float* gates;                                  // [tokens, 2 * heads]: delta (beta, g); mLSTM (i, f), logs;
                                                         // retention: [heads], the decay of each head
    float* out;                                          // [tokens, heads * vdim]
    float* state;                                        // this part's floats inside slot 0
    long long slot_stride;
    const int* span_begin; const int* span_slot;
    int heads, kv_heads, dim, vdim;
    float q_scale;
    int vector_copies;                                   // keys and queries can be staged 16 bytes at a time
};

__device__ __forceinline__ void cp_async_4(void* smem, const void* global) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(global));
}
__device__ __forceinline__ void cp_async_16(void* smem, const void* global) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(global));
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Four warps a block; a column of S lives in L lanes of 8 elements each (L = 1 .. 32 by the key size), so a warp
// holds 32 / L columns and a block four times as many. Element e of a column sits in lane (e / 4) % L, register
// 4 * (e / (4 L)) + e % 4: the lanes of a column read consecutive 16-byte pieces of a key. Few elements a lane keep
// the chain of dependent operations per token short (the sums meet by log2 L shuffles), and many warps keep the
// SMs busy when a step brings one long prompt.
template <int MODE, int L>
__global__ void __launch_bounds__(kScanThreads) recurrent_scan_kernel(const ScanParams p) {
    constexpr int kColsWarp = 32 / L;
    constexpr int kCols = kScanWarps * kColsWarp;
    constexpr int kDimPad = kScanRegs * L;
    constexpr int kTile = kDimPad > 128 ? 8 : 16;       // tokens staged at a time
    __shared__ __align__(16) float k_s[2][kTile][kDimPad];
    __shared__ __align__(16) float q_s[2][kTile][kDimPad];
    __shared__ float v_s[2][kTile][kCols];
    __shared__ float g_s[2][kTile][2];
    chain_release();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane % L, col_in = warp * kColsWarp + lane / L;
    const int head = blockIdx.y, span = blockIdx.z;
    const int kv_head = head / (p.heads / p.kv_heads);
    const int col = blockIdx.x * kCols + col_in;
    const bool col_ok = col < p.vdim;
    const int dim = p.dim, vdim = p.vdim;
    // keys beyond the head's size stay zero for good
    for (int i = tid; i < 2 * kTile * kDimPad; i += kScanThreads) {
        (&k_s[0][0][0])[i] = 0.0f;
        (&q_s[0][0][0])[i] = 0.0f;
    }
    for (int i = tid; i < 2 * kTile * kCols; i += kScanThreads) (&v_s[0][0][0])[i] = 0.0f;
    __syncthreads();
    chain_wait();
    const int t_begin = p.span_begin[span], t_end = p.span_begin[span + 1];
    if (t_end <= t_begin) return;
    float* slot = p.state + (long long)p.span_slot[span] * p.slot_stride;
    float* s_head = slot + (size_t)head * dim * vdim;
    float* n_head = slot + (size_t)p.heads * dim * vdim + (size_t)head * dim;
    float* m_head = slot + (size_t)p.heads * dim * vdim + (size_t)p.heads * dim + head;

    float s[kScanRegs], n[MODE == kScanMlstm ? kScanRegs : 1];
#pragma unroll
    for (int r = 0; r < kScanRegs; ++r) {
        const int e = 4 * ((r >> 2) * L + sub) + (r & 3);
        s[r] = (col_ok && e < dim) ? s_head[(size_t)e * vdim + col] : 0.0f;
        if (MODE == kScanMlstm) n[r] = e < dim ? n_head[e] : 0.0f;
    }
    float m = MODE == kScanMlstm ? *m_head : 0.0f;

    const float* k_base = p.k + (size_t)kv_head * dim;
    const float* q_base = p.q + (size_t)(MODE == kScanDelta ? kv_head : head) * dim;
    const float head_decay = MODE == kScanRetention ? p.gates[head] : 0.0f;
    auto issue = [&](int t0, int stage) {
        const int count = min(kTile, t_end - t0);
        if (p.vector_copies) {
            const int quads = dim >> 2;
            for (int i = tid; i < count * quads; i += kScanThreads) {
                const int tt = i / quads, e = (i - tt * quads) << 2;
                cp_async_16(&k_s[stage][tt][e], k_base + (size_t)(t0 + tt) * p.k_stride + e);
                cp_async_16(&q_s[stage][tt][e], q_base + (size_t)(t0 + tt) * p.q_stride + e);
            }
        } else {
            for (int i = tid; i < count * dim; i += kScanThreads) {
                const int tt = i / dim, e = i - tt * dim;
                cp_async_4(&k_s[stage][tt][e], k_base + (size_t)(t0 + tt) * p.k_stride + e);
                cp_async_4(&q_s[stage][tt][e], q_base + (size_t)(t0 + tt) * p.q_stride + e);
            }
        }
        for (int i = tid; i < count * kCols; i += kScanThreads) {
            const int tt = i / kCols, c = i % kCols;
            const int gc = blockIdx.x * kCols + c;
            if (gc < vdim) cp_async_4(&v_s[stage][tt][c], p.v + (size_t)(t0 + tt) * p.v_stride + (size_t)head * vdim + gc);
        }
        if (MODE != kScanRetention)
        for (int i = tid; i < count * 2; i += kScanThreads) {
            const int tt = i >> 1, w = i & 1;
            cp_async_4(&g_s[stage][tt][w], p.gates + (size_t)(t0 + tt) * 2 * p.heads + w * p.heads + head);
        }
        cp_async_commit_group();
    };

    issue(t_begin, 0);
    int stage = 0;
    for (int t0 = t_begin; t0 < t_end; t0 += kTile, stage ^= 1) {
        if (t0 + kTile < t_end) {
            issue(t0 + kTile, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                                // every thread's copies of this stage have landed
        const int count = min(kTile, t_end - t0);
#pragma unroll 4
        for (int tt = 0; tt < count; ++tt) {
            float kk[kScanRegs], qq[kScanRegs];
#pragma unroll
            for (int r4 = 0; r4 < kScanRegs / 4; ++r4) {
                const float4 kv4 = *reinterpret_cast<const float4*>(&k_s[stage][tt][4 * (r4 * L + sub)]);
                const float4 qv4 = *reinterpret_cast<const float4*>(&q_s[stage][tt][4 * (r4 * L + sub)]);
                kk[4 * r4] = kv4.x; kk[4 * r4 + 1] = kv4.y; kk[4 * r4 + 2] = kv4.z; kk[4 * r4 + 3] = kv4.w;
                qq[4 * r4] = qv4.x; qq[4 * r4 + 1] = qv4.y; qq[4 * r4 + 2] = qv4.z; qq[4 * r4 + 3] = qv4.w;
            }
            // sums over this lane's elements on the OLD state, in four partial sums each
            float sk[4] = {0.f, 0.f, 0.f, 0.f}, sq[4] = {0.f, 0.f, 0.f, 0.f}, kq[4] = {0.f, 0.f, 0.f, 0.f};
            float nq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < kScanRegs; ++r) {
                if (MODE == kScanDelta) sk[r & 3] = fmaf(s[r], kk[r], sk[r & 3]);
                sq[r & 3] = fmaf(s[r], qq[r], sq[r & 3]);
                kq[r & 3] = fmaf(kk[r], qq[r], kq[r & 3]);
                if (MODE == kScanMlstm) nq[r & 3] = fmaf(n[r], qq[r], nq[r & 3]);
            }
            float d_sk = (sk[0] + sk[1]) + (sk[2] + sk[3]);
            float d_sq = (sq[0] + sq[1]) + (sq[2] + sq[3]);
            float d_kq = (kq[0] + kq[1]) + (kq[2] + kq[3]);
            float d_nq = (nq[0] + nq[1]) + (nq[2] + nq[3]);
#pragma unroll
            for (int offset = 1; offset < L; offset <<= 1) {
                if (MODE == kScanDelta) d_sk += __shfl_xor_sync(0xffffffffu, d_sk, offset);
                d_sq += __shfl_xor_sync(0xffffffffu, d_sq, offset);
                d_kq += __shfl_xor_sync(0xffffffffu, d_kq, offset);
                if (MODE == kScanMlstm) d_nq += __shfl_xor_sync(0xffffffffu, d_nq, offset);
            }
            if (MODE != kScanRetention) d_sq *= p.q_scale;      // (retention: the factor is the key's, so S holds it)
            d_kq *= p.q_scale;
            d_nq *= p.q_scale;
            const float vj = v_s[stage][tt][col_in];
            const float g0 = MODE == kScanRetention ? 0.0f : g_s[stage][tt][0];
            const float g1 = MODE == kScanRetention ? 0.0f : g_s[stage][tt][1];
            float o;
            if (MODE == kScanRetention) {
                o = fmaf(head_decay, d_sq, vj * d_kq);
                const float vs = vj * p.q_scale;
#pragma unroll
                for (int r = 0; r < kScanRegs; ++r) s[r] = fmaf(kk[r], vs, head_decay * s[r]);
            } else if (MODE == kScanDelta) {
                const float beta = g0, decay = g1;
                const float u = beta * (vj - decay * d_sk);
                o = decay * d_sq + u * d_kq;
#pragma unroll
                for (int r = 0; r < kScanRegs; ++r) s[r] = fmaf(kk[r], u, decay * s[r]);
            } else {
                const float m_new = fmaxf(g1 + m, g0);
                const float keep = expf(g1 + m - m_new), write = expf(g0 - m_new);
                m = m_new;
                const float bv = write * vj;
                const float upper = keep * d_sq + bv * d_kq;
                const float lower = fmaxf(fabsf(keep * d_nq + write * d_kq), expf(-m_new)) + 1e-6f;
                o = upper / lower;
#pragma unroll
                for (int r = 0; r < kScanRegs; ++r) {
                    s[r] = fmaf(kk[r], bv, keep * s[r]);
                    n[r] = fmaf(kk[r], write, keep * n[r]);
                }
            }
            if (sub == 0 && col_ok) p.out[(size_t)(t0 + tt) * p.heads * vdim + (size_t)head * vdim + col] = o;
        }
        __syncthreads();                                // the stage is free for the tile after the next
    }
#pragma unroll
    for (int r = 0; r < kScanRegs; ++r) {
        const int e = 4 * ((r >> 2) * L + sub) + (r & 3);
        if (col_ok && e < dim) s_head[(size_t)e * vdim + col] = s[r];
        if (MODE == kScanMlstm && blockIdx.x == 0 && col_in == 0 && e < dim) n_head[e] = n[r];
    }
    if (MODE == kScanMlstm && blockIdx.x == 0 && tid == 0) *m_head = m;
}

// mLSTM: log input gate cap tanh((x_i + b_i) / cap) and log forget gate logsigmoid(cap tanh((x_f + b_f) / cap))
__global__ void mlstm_gates_kernel(const float* pre_i, const float* pre_f, int stride, const float* bias_i,
                                   const float* bias_f, float cap, float* gates, int tokens, int heads) {
    chain_release();
    chain_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= tokens * heads) return;
    const int t = i / heads, h = i % heads;
    const float gi = cap * tanhf((pre_i[(size_t)t * stride + h] + bias_i[h]) / cap);
    const float z = cap * tanhf((pre_f[(size_t)t * stride + h] + bias_f[h]) / cap);
    // logsigmoid(z) = min(z, 0) - log1p(exp(-|z|))
    const float gf = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
    gates[(size_t)t * 2 * heads + h] = gi;
    gates[(size_t)t * 2 * heads + heads + h] = gf;
}

struct DeltaPrepareArgs {
    const float* proj; int stride;          // rows [q | k | v | ...]: the first `channels` columns are convolved
    const float* kernel;                    // [channels, taps], the last tap multiplies the token itself
    const float* carried;                   // this part's carried inputs inside slot 0: [taps - 1, channels], oldest first
    long long slot_stride;
    const int* token_span; const int* span_begin; const int* span_slot;
    float* conv_out;                        // [tokens, channels]: silu(conv); q and k heads made unit vectors
    const float* pre_beta; const float* pre_a; int gate_stride;
    const float* a_log; const float* dt_bias;
    float* gates;                           // [tokens, 2 * heads]: beta, decay
    int tokens, channels, taps, qk_heads, dim, heads;
    float unit_eps;
    int vector_loads;                       // channels, strides and pointers allow 16-byte accesses
};

// One block a token: the three short convolutions with SiLU, then q and k per head divided by
// sqrt(sum of squares + eps), then beta = sigmoid(.) and decay = exp(-exp(A_log) softplus(. + dt_bias)).
__global__ void delta_prepare_kernel(const DeltaPrepareArgs a) {
    extern __shared__ float row[];          // [channels]
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int span = a.token_span[t];
    const int begin = a.span_begin[span];
    const float* carried = a.carried + (long long)a.span_slot[span] * a.slot_stride;
    const int rel = t - begin;
    if (a.vector_loads) {
        // four channels a thread, 16 bytes a load: all taps' loads of a thread are in flight together
        for (int c = 4 * threadIdx.x; c < a.channels; c += 4 * blockDim.x) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (a.taps == 4) {
                // four taps: a channel's kernel is one 16-byte load, and all eight loads are in flight together
                float4 x[4], w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int s = rel - 3 + j;
                    x[j] = *reinterpret_cast<const float4*>(s >= 0 ? a.proj + (size_t)(begin + s) * a.stride + c
                                                                   : carried + (size_t)(3 + s) * a.channels + c);
                    w[j] = __ldg(reinterpret_cast<const float4*>(a.kernel + (size_t)(c + j) * 4));
                }
                // (the same order of additions as the general loop: tap 0 first)
                sum.x = fmaf(w[0].w, x[3].x, fmaf(w[0].z, x[2].x, fmaf(w[0].y, x[1].x, w[0].x * x[0].x)));
                sum.y = fmaf(w[1].w, x[3].y, fmaf(w[1].z, x[2].y, fmaf(w[1].y, x[1].y, w[1].x * x[0].y)));
                sum.z = fmaf(w[2].w, x[3].z, fmaf(w[2].z, x[2].z, fmaf(w[2].y, x[1].z, w[2].x * x[0].z)));
                sum.w = fmaf(w[3].w, x[3].w, fmaf(w[3].z, x[2].w, fmaf(w[3].y, x[1].w, w[3].x * x[0].w)));
            } else
            for (int j = 0; j < a.taps; ++j) {
                const int s = rel - (a.taps - 1) + j;
                const float4 x = *reinterpret_cast<const float4*>(
                    s >= 0 ? a.proj + (size_t)(begin + s) * a.stride + c
                           : carried + (size_t)(a.taps - 1 + s) * a.channels + c);
                const float* w = a.kernel + (size_t)c * a.taps + j;
                sum.x = fmaf(__ldg(w), x.x, sum.x);
                sum.y = fmaf(__ldg(w + a.taps), x.y, sum.y);
                sum.z = fmaf(__ldg(w + 2 * a.taps), x.z, sum.z);
                sum.w = fmaf(__ldg(w + 3 * a.taps), x.w, sum.w);
            }
            row[c] = sum.x / (1.0f + expf(-sum.x));
            row[c + 1] = sum.y / (1.0f + expf(-sum.y));
            row[c + 2] = sum.z / (1.0f + expf(-sum.z));
            row[c + 3] = sum.w / (1.0f + expf(-sum.w));
        }
    } else {
        for (int c = threadIdx.x; c < a.channels; c += blockDim.x) {
            float sum = 0.0f;
            for (int j = 0; j < a.taps; ++j) {
                const int s = rel - (a.taps - 1) + j;
                const float x = s >= 0 ? a.proj[(size_t)(begin + s) * a.stride + c]
                                       : carried[(size_t)(a.taps - 1 + s) * a.channels + c];
                sum = fmaf(a.kernel[(size_t)c * a.taps + j], x, sum);
            }
            row[c] = sum / (1.0f + expf(-sum));
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int h = warp; h < 2 * a.qk_heads; h += warps) {     // q heads, then k heads
        float sum = 0.0f;
        for (int i = lane; i < a.dim; i += 32) sum += row[h * a.dim + i] * row[h * a.dim + i];
        sum = warp_sum(sum);
        const float inv = 1.0f / sqrtf(sum + a.unit_eps);
        for (int i = lane; i < a.dim; i += 32) row[h * a.dim + i] *= inv;
    }
    __syncthreads();
    float* dst = a.conv_out + (size_t)t * a.channels;
    if (a.vector_loads) {
        for (int c = 4 * threadIdx.x; c < a.channels; c += 4 * blockDim.x)
            *reinterpret_cast<float4*>(dst + c) = make_float4(row[c], row[c + 1], row[c + 2], row[c + 3]);
    } else {
        for (int c = threadIdx.x; c < a.channels; c += blockDim.x) dst[c] = row[c];
    }
    for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
        const float b = a.pre_beta[(size_t)t * a.gate_stride + h];
        const float x = a.pre_a[(size_t)t * a.gate_stride + h] + a.dt_bias[h];
        const float soft = fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x)));
        a.gates[(size_t)t * 2 * a.heads + h] = 1.0f / (1.0f + expf(-b));
        a.gates[(size_t)t * 2 * a.heads + a.heads + h] = expf(-expf(a.a_log[h]) * soft);
    }
}

// The carried inputs after a step: the last taps - 1 inputs of each request's sequence. One thread per
// (span, channel) reads everything it needs before it writes, so the update is in place.
__global__ void carried_inputs_update_kernel(const float* proj, int stride, float* carried, long long slot_stride,
                                             const int* span_begin, const int* span_slot, int spans, int channels,
                                             int taps) {
    chain_release();
    chain_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= spans * channels) return;
    const int span = i / channels, c = i % channels;
    const int begin = span_begin[span], len = span_begin[span + 1] - begin;
    float* mine = carried + (long long)span_slot[span] * slot_stride;
    float keep[15];
#pragma unroll
    for (int r = 0; r < 15; ++r) {
        if (r < taps - 1) {
            const int s = len - (taps - 1) + r;
            keep[r] = s >= 0 ? proj[(size_t)(begin + s) * stride + c] : mine[(size_t)(taps - 1 + s) * channels + c];
        }
    }
#pragma unroll
    for (int r = 0; r < 15; ++r)
        if (r < taps - 1) mine[(size_t)r * channels + c] = keep[r];
}

// One warp per (token, head): o / sqrt(mean(o^2) + eps) * w * act(gate), act = sigmoid (0) or SiLU (1);
// w is [heads * vdim] or, shared by the heads, [vdim].
template <typename A>
__global__ void gated_head_norm_kernel(const float* o, const float* gate, int gate_stride, const float* weight,
                                       int weight_per_head, A* out, int tokens, int heads, int vdim, float eps,
                                       int gate_kind) {
    chain_release();
    chain_wait();
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)tokens * heads) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(unit / heads), h = (int)(unit % heads);
    const float* src = o + ((size_t)t * heads + h) * vdim;
    float sum = 0.0f;
    for (int i = lane; i < vdim; i += 32) sum += src[i] * src[i];
    sum = warp_sum(sum);
    const float inv = 1.0f / sqrtf(sum / (float)vdim + eps);
    const float* w = weight ? weight + (weight_per_head ? (size_t)h * vdim : 0) : nullptr;     // (null: no weight)
    const float* g = gate + (size_t)t * gate_stride + (size_t)h * vdim;
    A* dst = out + ((size_t)t * heads + h) * vdim;
    for (int i = lane; i < vdim; i += 32) {
        const float z = g[i];
        const float sig = 1.0f / (1.0f + expf(-z));
        dst[i] = from_float<A>(src[i] * inv * (w ? w[i] : 1.0f) * (gate_kind == 0 ? sig : z * sig));
    }
}

// The same for wide units (one norm over all heads' columns together): a block per (token, head), 16-byte reads
// where the rows allow them. The order of the sum differs from the warp's; both are float32 sums of the same squares.
template <typename A>
__global__ void __launch_bounds__(256) gated_row_norm_kernel(const float* o, const float* gate, int gate_stride,
                                                             const float* weight, int weight_per_head, A* out, int heads,
                                                             int vdim, float eps, int gate_kind, int vectors) {
    __shared__ float partial[8];
    chain_release();
    chain_wait();
    const long long unit = blockIdx.x;
    const int t = (int)(unit / heads), h = (int)(unit % heads);
    const float* src = o + ((size_t)t * heads + h) * vdim;
    const float* w = weight ? weight + (weight_per_head ? (size_t)h * vdim : 0) : nullptr;
    const float* g = gate + (size_t)t * gate_stride + (size_t)h * vdim;
    A* dst = out + ((size_t)t * heads + h) * vdim;
    float sum = 0.0f;
    if (vectors) {
        for (int i = threadIdx.x * 4; i < vdim; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < vdim; i += blockDim.x) sum += src[i] * src[i];
    }
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
    __syncthreads();
    sum = 0.0f;
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) sum += partial[k];      // (every thread adds in the same order)
    const float inv = 1.0f / sqrtf(sum / (float)vdim + eps);
    auto one = [&](float x, float z, float scale) {
        const float sig = 1.0f / (1.0f + expf(-z));
        return x * inv * scale * (gate_kind == 0 ? sig : z * sig);
    };
    if (vectors) {
        for (int i = threadIdx.x * 4; i < vdim; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            const float4 z = *reinterpret_cast<const float4*>(g + i);
            const float4 s = w ? *reinterpret_cast<const float4*>(w + i) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            dst[i] = from_float<A>(one(v.x, z.x, s.x));
            dst[i + 1] = from_float<A>(one(v.y, z.y, s.y));
            dst[i + 2] = from_float<A>(one(v.z, z.z, s.z));
            dst[i + 3] = from_float<A>(one(v.w, z.w, s.w));
        }
    } else {
        for (int i = threadIdx.x; i < vdim; i += blockDim.x) dst[i] = from_float<A>(one(src[i], g[i], w ? w[i] : 1.0f));
    }
}

// ---------------------------------------------------------------------------------------------------------
// Decoding: every request brings one token. One block per (request, head) does everything between the input
// projection and the output projection: the delta rule's short convolutions over the carried inputs with SiLU,
// unit q and k, beta and decay (or the mLSTM's two gates), the state's update and read-out with a thread per
// column (rows of S are read and written side by side: whole lines of memory), the head's root mean square, the
// norm's weight and the output gate. Same formulas and the same sums on the old state as the scan above.
struct DecodeStepParams {
    const float* proj; int stride;                 // [tokens, stride] rows of the input projection
    int q_off, k_off, v_off, gate_off, g0_off, g1_off;
    const float* conv_kernel; const float* carried; int taps, channels;      // delta only
    const float* bias0; const float* bias1; float cap;   // mLSTM: gate biases and cap; delta: A_log and dt_bias
    const float* norm_w; int norm_per_head; float eps, unit_eps;
    float* state; long long slot_stride;
    const int* span_slot;
    int heads, kv_heads, dim, vdim;
    float q_scale;
    void* out;                                     // [tokens, heads * vdim], activation type
    int input_act;                                 // retention, mLSTM: an activation of q, k and v as read (-1: none)
    float* raw_out;                                // not null: the read-outs go here as they are, float32 [tokens,
                                                   // heads * vdim], and norm and gate are the caller's (one over all heads)
};

template <int MODE, typename A>
__global__ void __launch_bounds__(256) recurrent_decode_kernel(const DecodeStepParams p) {
    extern __shared__ float decode_smem[];          // k [dim] | q [dim] | o [vdim] | partial sums [2 * warps * 32]
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int head = blockIdx.x, t = blockIdx.y;
    const int dim = p.dim, vdim = p.vdim, heads = p.heads;
    const int kv_head = head / (heads / p.kv_heads);
    const int qk_head = MODE == kScanDelta ? kv_head : head;
    float* k_s = decode_smem;
    float* q_s = k_s + dim;
    float* o_s = q_s + dim;
    float* part_s = o_s + vdim;
    const float* row = p.proj + (size_t)t * p.stride;
    const long long slot_at = (long long)p.span_slot[t] * p.slot_stride;
    const float* carried = MODE == kScanDelta ? p.carried + slot_at : nullptr;

    // a convolved channel of the delta rule: taps - 1 carried inputs (oldest first), then the token's own
    auto convolved = [&](int c) {
        float sum = 0.0f;
        for (int j = 0; j + 1 < p.taps; ++j)
            sum = fmaf(p.conv_kernel[(size_t)c * p.taps + j], carried[(size_t)j * p.channels + c], sum);
        sum = fmaf(p.conv_kernel[(size_t)c * p.taps + p.taps - 1], row[c], sum);
        return sum / (1.0f + expf(-sum));
    };
    float k2 = 0.0f, q2 = 0.0f;
    for (int e = threadIdx.x; e < dim; e += blockDim.x) {
        float kv, qv;
        if (MODE == kScanDelta) {
            kv = convolved(p.k_off + qk_head * dim + e);
            qv = convolved(p.q_off + qk_head * dim + e);
        } else {
            kv = row[p.k_off + qk_head * dim + e];
            qv = row[p.q_off + qk_head * dim + e];
            if (p.input_act >= 0) {
                kv = activate(kv, p.input_act);
                qv = activate(qv, p.input_act);
            }
        }
        k_s[e] = kv;
        q_s[e] = qv;
        k2 += kv * kv;
        q2 += qv * qv;
    }
    if (MODE == kScanDelta) {
        k2 = block_sum(k2, scratch);
        q2 = block_sum(q2, scratch);
        const float k_inv = 1.0f / sqrtf(k2 + p.unit_eps), q_inv = 1.0f / sqrtf(q2 + p.unit_eps);
        for (int e = threadIdx.x; e < dim; e += blockDim.x) {
            k_s[e] *= k_inv;
            q_s[e] *= q_inv;
        }
    }
    __syncthreads();
    float* slot = p.state + slot_at;
    float* s_head = slot + (size_t)head * dim * vdim;
    float* n_head = slot + (size_t)heads * dim * vdim + (size_t)head * dim;
    float* m_head = slot + (size_t)heads * dim * vdim + (size_t)heads * dim + head;
    float kq = 0.0f, nq = 0.0f;
    for (int e = threadIdx.x; e < dim; e += blockDim.x) {
        kq = fmaf(k_s[e], q_s[e], kq);
        if (MODE == kScanMlstm) nq = fmaf(n_head[e], q_s[e], nq);
    }
    kq = block_sum(kq, scratch) * p.q_scale;
    if (MODE == kScanMlstm) nq = block_sum(nq, scratch) * p.q_scale;

    float g0, g1, keep = 0.0f, write = 0.0f, lower = 1.0f, m_new = 0.0f;
    if (MODE == kScanRetention) {
        g0 = 1.0f;
        g1 = p.bias0[head];                                                     // the head's decay
    } else if (MODE == kScanDelta) {
        g0 = 1.0f / (1.0f + expf(-row[p.g0_off + head]));                      // beta
        const float x = row[p.g1_off + head] + p.bias1[head];
        g1 = expf(-expf(p.bias0[head]) * (fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x)))));     // decay
    } else {
        g0 = p.cap * tanhf((row[p.g0_off + head] + p.bias0[head]) / p.cap);     // log input gate
        const float z = p.cap * tanhf((row[p.g1_off + head] + p.bias1[head]) / p.cap);
        g1 = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));                          // log forget gate
        const float m = *m_head;
        m_new = fmaxf(g1 + m, g0);
        keep = expf(g1 + m - m_new);
        write = expf(g0 - m_new);
        lower = fmaxf(fabsf(keep * nq + write * kq), expf(-m_new)) + 1e-6f;
    }
    // The state: a warp takes 32 neighbouring columns and every ``split``-th row of them, so that a block's warps
    // cover the head's columns with `split` warps each; a thread's rows stay in registers between the sums and
    // the update (up to 32 of them; beyond that they are read again), all of its loads are in flight at once, and
    // the partial sums of a column meet in shared memory.
    constexpr int kKeep = 32;
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = (vdim + 31) >> 5;
    const int split = max(1, warps / groups);
    const int groups_at_once = warps / split;
    const bool kept = dim <= kKeep * split;
    float squares = 0.0f;
    for (int first_group = 0; first_group < groups; first_group += groups_at_once) {
        const int g = first_group + warp / split, part = warp % split;
        const int j = g * 32 + lane;
        const bool active = warp < groups_at_once * split && g < groups && j < vdim;
        float cells[kKeep];
        float sk = 0.0f, sq = 0.0f;
        if (active) {
            if (kept) {
#pragma unroll
                for (int i = 0; i < kKeep; ++i) {
                    const int e = part + i * split;
                    cells[i] = e < dim ? s_head[(size_t)e * vdim + j] : 0.0f;
                }
#pragma unroll
                for (int i = 0; i < kKeep; ++i) {
                    const int e = part + i * split;
                    if (e < dim) {
                        if (MODE == kScanDelta) sk = fmaf(cells[i], k_s[e], sk);
                        sq = fmaf(cells[i], q_s[e], sq);
                    }
                }
            } else {
                for (int e = part; e < dim; e += split) {
                    const float se = s_head[(size_t)e * vdim + j];
                    if (MODE == kScanDelta) sk = fmaf(se, k_s[e], sk);
                    sq = fmaf(se, q_s[e], sq);
                }
            }
        }
        __syncthreads();                              // (the partial sums of the pass before have been read)
        part_s[warp * 32 + lane] = sk;
        part_s[(warps + warp) * 32 + lane] = sq;
        __syncthreads();
        if (active) {
            sk = sq = 0.0f;
            const int first = (warp / split) * split;
            for (int w = first; w < first + split; ++w) {
                sk += part_s[w * 32 + lane];
                sq += part_s[(warps + w) * 32 + lane];
            }
            if (MODE != kScanRetention) sq *= p.q_scale;
            float vj = MODE == kScanDelta ? convolved(p.v_off + head * vdim + j) : row[p.v_off + head * vdim + j];
            if (MODE != kScanDelta && p.input_act >= 0) vj = activate(vj, p.input_act);
            float o, scale, add;
            if (MODE == kScanRetention) {
                add = vj * p.q_scale;                 // the key's factor: S holds scaled keys
                scale = g1;
                o = fmaf(g1, sq, vj * kq);
            } else if (MODE == kScanDelta) {
                add = g0 * (vj - g1 * sk);            // u
                scale = g1;
                o = g1 * sq + add * kq;
            } else {
                add = write * vj;
                scale = keep;
                o = (keep * sq + add * kq) / lower;
            }
            if (kept) {
#pragma unroll
                for (int i = 0; i < kKeep; ++i) {
                    const int e = part + i * split;
                    if (e < dim) s_head[(size_t)e * vdim + j] = fmaf(k_s[e], add, scale * cells[i]);
                }
            } else {
                for (int e = part; e < dim; e += split) {
                    float* cell = s_head + (size_t)e * vdim + j;
                    *cell = fmaf(k_s[e], add, scale * *cell);
                }
            }
            if (part == 0) {
                o_s[j] = o;
                squares += o * o;
            }
        }
    }
    if (MODE == kScanMlstm) {
        __syncthreads();                              // every thread has read n and m
        for (int e = threadIdx.x; e < dim; e += blockDim.x) n_head[e] = fmaf(k_s[e], write, keep * n_head[e]);
        if (threadIdx.x == 0) *m_head = m_new;
    }
    if (p.raw_out) {
        __syncthreads();
        float* raw = p.raw_out + ((size_t)t * heads + head) * vdim;
        for (int j = threadIdx.x; j < vdim; j += blockDim.x) raw[j] = o_s[j];
        return;
    }
    squares = block_sum(squares, scratch);
    const float inv = 1.0f / sqrtf(squares / (float)vdim + p.eps);
    const float* w = p.norm_w ? p.norm_w + (p.norm_per_head ? (size_t)head * vdim : 0) : nullptr;   // (null: no weight)
    A* dst = static_cast<A*>(p.out) + ((size_t)t * heads + head) * vdim;
    for (int j = threadIdx.x; j < vdim; j += blockDim.x) {
        const float z = row[p.gate_off + head * vdim + j];
        const float sig = 1.0f / (1.0f + expf(-z));
        dst[j] = from_float<A>(o_s[j] * inv * (w ? w[j] : 1.0f) * (MODE == kScanMlstm ? sig : z * sig));
    }
}

// ---------------------------------------------------------------------------------------------------------
// Retention over long spans, cut into segments. With a constant decay d the state after token t of a segment
// that begins at token b is S_t = d^(t-b+1) S_(b-1) + L_t, L_t the state the segment's own tokens would have built
// from zero. So the segments of all spans are scanned side by side from zero states (the scan kernel above, one
// "span" a segment), which also gives the segment's final L and the local read-outs L_t^T q_t; the states at the
// segments' starts follow from one another by S <- d^len S + L (a handful of steps a span, element by element);
// and the read-outs get d^(t-b+1) S_(b-1)^T q_t added, a small product per segment. Only rounding differs
// from the token-by-token order.
// The segments' scan, built for throughput instead of a short chain per token (many segments run side by side, so
// no single one is waited for): a lane holds 64 consecutive elements of a column of S (the whole column up to a key
// size of 64; L = 2 or 4 lanes a column beyond), reads a token's key and query as 16-byte broadcasts from shared
// memory, and k.q is formed once per token for all columns. Per element and token that is a third of the
// instructions of the kernel above, which spreads a column over eight lanes to keep ONE long span's chain short.
template <int L>
__global__ void __launch_bounds__(kScanThreads) retention_wide_scan_kernel(const ScanParams p) {
    constexpr int kE = 64;
    constexpr int kColsWarp = 32 / L;
    constexpr int kCols = kScanWarps * kColsWarp;
    constexpr int kDimPad = kE * L;
    constexpr int kTile = L > 2 ? 8 : 16;
    __shared__ __align__(16) float k_s[2][kTile][kDimPad];
    __shared__ __align__(16) float q_s[2][kTile][kDimPad];
    __shared__ float v_s[2][kTile][kCols];
    __shared__ float kq_s[2][kTile];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane % L, col_in = warp * kColsWarp + lane / L;
    const int head = blockIdx.y, span = blockIdx.z;
    const int col = blockIdx.x * kCols + col_in;
    const bool col_ok = col < p.vdim;
    const int dim = p.dim, vdim = p.vdim;
    const int t_begin = p.span_begin[span], t_end = p.span_begin[span + 1];
    if (t_end <= t_begin) return;
    for (int i = tid; i < 2 * kTile * kDimPad; i += kScanThreads) {      // keys beyond the head's size stay zero
        (&k_s[0][0][0])[i] = 0.0f;
        (&q_s[0][0][0])[i] = 0.0f;
    }
    for (int i = tid; i < 2 * kTile * kCols; i += kScanThreads) (&v_s[0][0][0])[i] = 0.0f;
    __syncthreads();
    float* s_head = p.state + (long long)p.span_slot[span] * p.slot_stride + (size_t)head * dim * vdim;
    const float decay = p.gates[head];
    float s[kE];
#pragma unroll
    for (int r = 0; r < kE; ++r) {
        const int e = sub * kE + r;
        s[r] = (col_ok && e < dim) ? s_head[(size_t)e * vdim + col] : 0.0f;
    }
    const float* k_base = p.k + (size_t)head * dim;
    const float* q_base = p.q + (size_t)head * dim;
    auto issue = [&](int t0, int stage) {
        const int count = min(kTile, t_end - t0);
        if (p.vector_copies) {
            const int quads = dim >> 2;
            for (int i = tid; i < count * quads; i += kScanThreads) {
                const int tt = i / quads, e = (i - tt * quads) << 2;
                cp_async_16(&k_s[stage][tt][e], k_base + (size_t)(t0 + tt) * p.k_stride + e);
                cp_async_16(&q_s[stage][tt][e], q_base + (size_t)(t0 + tt) * p.q_stride + e);
            }
        } else {
            for (int i = tid; i < count * dim; i += kScanThreads) {
                const int tt = i / dim, e = i - tt * dim;
                cp_async_4(&k_s[stage][tt][e], k_base + (size_t)(t0 + tt) * p.k_stride + e);
                cp_async_4(&q_s[stage][tt][e], q_base + (size_t)(t0 + tt) * p.q_stride + e);
            }
        }
        for (int i = tid; i < count * kCols; i += kScanThreads) {
            const int tt = i / kCols, c = i % kCols;
            const int gc = blockIdx.x * kCols + c;
            if (gc < vdim) cp_async_4(&v_s[stage][tt][c], p.v + (size_t)(t0 + tt) * p.v_stride + (size_t)head * vdim + gc);
        }
        cp_async_commit_group();
    };
    issue(t_begin, 0);
    int stage = 0;
    for (int t0 = t_begin; t0 < t_end; t0 += kTile, stage ^= 1) {
        if (t0 + kTile < t_end) {
            issue(t0 + kTile, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                                // every thread's copies of this stage have landed
        const int count = min(kTile, t_end - t0);
        for (int tt = warp; tt < count; tt += kScanWarps) {            // k.q of the tile's tokens, a warp a token
            float sum = 0.0f;
            for (int e = lane; e < kDimPad; e += 32) sum = fmaf(k_s[stage][tt][e], q_s[stage][tt][e], sum);
            sum = warp_sum(sum);
            if (lane == 0) kq_s[stage][tt] = sum * p.q_scale;
        }
        __syncthreads();
        for (int tt = 0; tt < count; ++tt) {
            const float vj = v_s[stage][tt][col_in];
            const float vs = vj * p.q_scale;
            const float4* kp = reinterpret_cast<const float4*>(&k_s[stage][tt][sub * kE]);
            const float4* qp = reinterpret_cast<const float4*>(&q_s[stage][tt][sub * kE]);
            float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int r4 = 0; r4 < kE / 4; ++r4) {
                const float4 kv = kp[r4], qv = qp[r4];
                sq[0] = fmaf(s[4 * r4], qv.x, sq[0]);
                sq[1] = fmaf(s[4 * r4 + 1], qv.y, sq[1]);
                sq[2] = fmaf(s[4 * r4 + 2], qv.z, sq[2]);
                sq[3] = fmaf(s[4 * r4 + 3], qv.w, sq[3]);
                s[4 * r4] = fmaf(kv.x, vs, decay * s[4 * r4]);
                s[4 * r4 + 1] = fmaf(kv.y, vs, decay * s[4 * r4 + 1]);
                s[4 * r4 + 2] = fmaf(kv.z, vs, decay * s[4 * r4 + 2]);
                s[4 * r4 + 3] = fmaf(kv.w, vs, decay * s[4 * r4 + 3]);
            }
            float d_sq = (sq[0] + sq[1]) + (sq[2] + sq[3]);
#pragma unroll
            for (int offset = 1; offset < L; offset <<= 1) d_sq += __shfl_xor_sync(0xffffffffu, d_sq, offset);
            if (sub == 0 && col_ok)
                p.out[(size_t)(t0 + tt) * p.heads * vdim + (size_t)head * vdim + col] = fmaf(decay, d_sq, vj * kq_s[stage][tt]);
        }
        __syncthreads();                                // the stage is free for the tile after the next
    }
#pragma unroll
    for (int r = 0; r < kE; ++r) {
        const int e = sub * kE + r;
        if (col_ok && e < dim) s_head[(size_t)e * vdim + col] = s[r];
    }
}

static int launch_wide_scan(const ScanParams& p, int spans, cudaStream_t stream) {
    const int lanes = p.dim <= 64 ? 1 : p.dim <= 128 ? 2 : 4;
    const int cols = kScanWarps * (32 / lanes);
    dim3 grid((p.vdim + cols - 1) / cols, p.heads, spans);
    if (lanes == 1) retention_wide_scan_kernel<1><<<grid, kScanThreads, 0, stream>>>(p);
    else if (lanes == 2) retention_wide_scan_kernel<2><<<grid, kScanThreads, 0, stream>>>(p);
    else retention_wide_scan_kernel<4><<<grid, kScanThreads, 0, stream>>>(p);
    return check_launch("retention_wide_scan");
}

__global__ void retention_plan_kernel(const int* span_begin, int spans, int segment, int max_segments, int* seg_begin,
                                      int* span_first) {
    chain_release();
    chain_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int n = 0;
    for (int s = 0; s < spans; ++s) {
        span_first[s] = n;
        for (int b = span_begin[s]; b < span_begin[s + 1] && n < max_segments; b += segment) seg_begin[n++] = b;
    }
    span_first[spans] = n;
    for (int i = n; i <= max_segments; ++i) seg_begin[i] = span_begin[spans];      // (segments beyond the last are empty)
}

// one thread a state element: the state at every segment's start, and the span's state after its last token
__global__ void retention_carry_kernel(float* state, long long slot_stride, const int* span_slot, const int* span_first,
                                       const int* seg_begin, const float* local, float* carried, const float* decay,
                                       int elements, int head_elements) {
    chain_release();
    chain_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elements) return;
    const int span = blockIdx.y;
    float* cell = state + (long long)span_slot[span] * slot_stride + e;
    const float d = decay[e / head_elements];
    float s = *cell;
    for (int seg = span_first[span]; seg < span_first[span + 1]; ++seg) {
        carried[(size_t)seg * elements + e] = s;
        s = fmaf(powf(d, (float)(seg_begin[seg + 1] - seg_begin[seg])), s, local[(size_t)seg * elements + e]);
    }
    *cell = s;
}

// out[t, head, :] += d^(t - b + 1) (carried[segment of t][head]^T q_t): 64 tokens x 64 columns a block, FFMA
__global__ void __launch_bounds__(256) retention_add_carried_kernel(const float* q, int q_stride, const float* carried,
                                                                    const int* seg_begin, const float* decay, float* out,
                                                                    int heads, int dim, int vdim, int pieces) {
    __shared__ float qs[16][64 + 4];
    __shared__ float ss[16][64 + 4];
    chain_release();
    chain_wait();
    const int seg = blockIdx.z / pieces, piece = blockIdx.z % pieces;
    const int head = blockIdx.y, col0 = blockIdx.x * 64;
    const int begin = seg_begin[seg], end = seg_begin[seg + 1];
    const int t0 = begin + piece * 64;
    if (t0 >= end) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const float* state = carried + ((size_t)seg * heads + head) * dim * vdim;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < dim; k0 += 16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, kk = idx & 15;            // queries: 16 k of a token are neighbours
            qs[kk][r] = (t0 + r < end && k0 + kk < dim) ? q[(size_t)(t0 + r) * q_stride + (size_t)head * dim + k0 + kk] : 0.0f;
            const int c = idx & 63, kr = idx >> 6;            // state rows: 64 columns of a k are neighbours
            ss[kr][c] = (col0 + c < vdim && k0 + kr < dim) ? state[(size_t)(k0 + kr) * vdim + col0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = qs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ss[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    const float d = decay[head];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= end) continue;
        const float factor = powf(d, (float)(t - begin + 1));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx * 4 + j;
            if (c < vdim) {
                float* cell = out + (size_t)t * heads * vdim + (size_t)head * vdim + c;
                *cell = fmaf(factor, acc[i][j], *cell);
            }
        }
    }
}

template <int MODE>
static int launch_scan(const ScanParams& p, int spans, cudaStream_t stream) {
    int lanes = 1;
    while (lanes * kScanRegs < p.dim) lanes <<= 1;           // 1 .. 32 for key sizes up to 256
    const int cols = kScanWarps * (32 / lanes);
    dim3 grid((p.vdim + cols - 1) / cols, p.heads, spans);
    // A plain launch, not a chained one: a chained launch lets this kernel's few long-running blocks become resident
    // while the kernel before still fills the SMs, and they end up packed on the few SMs that had room (measured: a
    // prompt of 2,048 tokens took 9.6 ms with the scans chained and 5.2 ms without).
    switch (lanes) {
        case 1: recurrent_scan_kernel<MODE, 1><<<grid, kScanThreads, 0, stream>>>(p); break;
        case 2: recurrent_scan_kernel<MODE, 2><<<grid, kScanThreads, 0, stream>>>(p); break;
        case 4: recurrent_scan_kernel<MODE, 4><<<grid, kScanThreads, 0, stream>>>(p); break;
        case 8: recurrent_scan_kernel<MODE, 8><<<grid, kScanThreads, 0, stream>>>(p); break;
        case 16: recurrent_scan_kernel<MODE, 16><<<grid, kScanThreads, 0, stream>>>(p); break;
        default: recurrent_scan_kernel<MODE, (kScanMaxDim / kScanRegs >= 32 ? 32 : 16)><<<grid, kScanThreads, 0, stream>>>(p); break;
    }
    return check_launch("recurrent_scan");
}

}  // namespace celeg_b200

using namespace celeg_b200;

// mode 0: gated delta rule (q heads = kv_heads, gates = beta | decay); mode 1: mLSTM (q heads = heads,
// gates = log input | log forget; the slot holds S, then n [heads, dim], then m [heads]); mode 2: retention
// (q heads = heads, gates = one decay per head [heads]).
CELEG_API int celeg_recurrent_scan(int mode, const float* q, int q_stride, const float* k, int k_stride, const float* v,
                                   int v_stride, const float* gates, float* out, float* state, long long slot_stride,
                                   const int* span_begin, const int* span_slot, int spans, int heads, int kv_heads,
                                   int dim, int vdim, float q_scale, cudaStream_t stream) {
    CELEG_REQUIRE(spans >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0,
                  "recurrent_scan: invalid sizes spans=%d heads=%d kv_heads=%d dim=%d vdim=%d", spans, heads, kv_heads,
                  dim, vdim);
    CELEG_REQUIRE(dim <= kScanMaxDim, "recurrent_scan: a key size of %d exceeds %d", dim, kScanMaxDim);
    CELEG_REQUIRE(mode == kScanDelta || mode == kScanMlstm || mode == kScanRetention, "recurrent_scan: unknown mode %d", mode);
    CELEG_REQUIRE(spans <= 65535 && heads <= 65535, "recurrent_scan: %d spans or %d heads exceed one launch", spans, heads);
    if (spans == 0) return 0;
    const int vector_copies = dim % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 &&
                              (((size_t)q | (size_t)k) & 15) == 0;
    const ScanParams p = {q, k, v, q_stride, k_stride, v_stride, gates, out, state, slot_stride, span_begin, span_slot,
                          heads, kv_heads, dim, vdim, q_scale, vector_copies};
    if (mode == kScanRetention) return launch_scan<kScanRetention>(p, spans, stream);
    return mode == kScanDelta ? launch_scan<kScanDelta>(p, spans, stream) : launch_scan<kScanMlstm>(p, spans, stream);
}

CELEG_API int celeg_mlstm_gates(const float* pre_i, const float* pre_f, int stride, const float* bias_i,
                                const float* bias_f, float cap, float* gates, int tokens, int heads,
                                cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && heads > 0 && cap > 0.0f, "mlstm_gates: invalid sizes tokens=%d heads=%d cap=%g", tokens,
                  heads, cap);
    if (tokens == 0) return 0;
    const long long units = (long long)tokens * heads;
    launch_chained(mlstm_gates_kernel, (unsigned)((units + 127) / 128), 128, 0, stream, pre_i, pre_f, stride, bias_i,
                   bias_f, cap, gates, tokens, heads);
    return check_launch("mlstm_gates");
}

CELEG_API int celeg_delta_prepare(const float* proj, int stride, const float* kernel, float* carried,
                                  long long slot_stride, const int* token_span, const int* span_begin,
                                  const int* span_slot, float* conv_out, const float* pre_beta, const float* pre_a,
                                  const float* a_log, const float* dt_bias, float* gates, int tokens, int spans,
                                  int channels, int taps, int qk_heads, int dim, int heads, float unit_eps,
                                  cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && spans >= 0 && channels > 0 && taps >= 1 && taps <= 16 && qk_heads > 0 && dim > 0 &&
                  heads > 0 && 2 * qk_heads * dim <= channels,
                  "delta_prepare: invalid sizes tokens=%d channels=%d taps=%d qk_heads=%d dim=%d heads=%d", tokens,
                  channels, taps, qk_heads, dim, heads);
    CELEG_REQUIRE((size_t)channels * sizeof(float) <= 48 * 1024, "delta_prepare: %d channels exceed a block's shared memory",
                  channels);
    if (tokens == 0) return 0;
    DeltaPrepareArgs args = {proj, stride, kernel, carried, slot_stride, token_span, span_begin, span_slot,
                                   conv_out, pre_beta, pre_a, stride, a_log, dt_bias, gates, tokens, channels, taps,
                                   qk_heads, dim, heads, unit_eps, 0};
    args.vector_loads =
        channels % 4 == 0 && stride % 4 == 0 && slot_stride % 4 == 0 &&
        (((size_t)proj | (size_t)carried | (size_t)conv_out) & 15) == 0;
    launch_chained(delta_prepare_kernel, tokens, 256, (size_t)channels * sizeof(float), stream, args);
    int status = check_launch("delta_prepare");
    if (status != 0 || taps == 1) return status;
    const long long units = (long long)spans * channels;
    launch_chained(carried_inputs_update_kernel, (unsigned)((units + 127) / 128), 128, 0, stream, proj, stride, carried,
                   slot_stride, span_begin, span_slot, spans, channels, taps);
    return check_launch("carried_inputs_update");
}

CELEG_API int celeg_gated_head_norm(const float* o, const float* gate, int gate_stride, const float* weight,
                                    int weight_per_head, void* out, int tokens, int heads, int vdim, float eps,
                                    int gate_kind, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0 && eps > 0.0f && (gate_kind == 0 || gate_kind == 1),
                  "gated_head_norm: invalid sizes tokens=%d heads=%d vdim=%d eps=%g gate=%d", tokens, heads, vdim, eps,
                  gate_kind);
    if (tokens == 0) return 0;
    const long long units = (long long)tokens * heads;
    if (vdim >= 512) {          // a unit is worth a block
        CELEG_REQUIRE(units <= 0x7fffffffLL, "gated_head_norm: %lld units exceed one launch", units);
        const int vectors = vdim % 4 == 0 && gate_stride % 4 == 0 && ((uintptr_t)o | (uintptr_t)gate | (uintptr_t)weight) % 16 == 0;
        if (act_dtype == kFloat32)
            launch_chained(gated_row_norm_kernel<float>, (unsigned)units, 256, 0, stream, o, gate, gate_stride, weight,
                           weight_per_head, (float*)out, heads, vdim, eps, gate_kind, vectors);
        else if (act_dtype == kBFloat16)
            launch_chained(gated_row_norm_kernel<__nv_bfloat16>, (unsigned)units, 256, 0, stream, o, gate, gate_stride,
                           weight, weight_per_head, (__nv_bfloat16*)out, heads, vdim, eps, gate_kind, vectors);
        else
            CELEG_REQUIRE(false, "gated_head_norm: unknown dtype code %d", act_dtype);
        return check_launch("gated_head_norm");
    }
    const unsigned blocks = (unsigned)((units + 3) / 4);
    if (act_dtype == kFloat32)
        launch_chained(gated_head_norm_kernel<float>, blocks, 128, 0, stream, o, gate, gate_stride, weight,
                       weight_per_head, (float*)out, tokens, heads, vdim, eps, gate_kind);
    else if (act_dtype == kBFloat16)
        launch_chained(gated_head_norm_kernel<__nv_bfloat16>, blocks, 128, 0, stream, o, gate, gate_stride, weight,
                       weight_per_head, (__nv_bfloat16*)out, tokens, heads, vdim, eps, gate_kind);
    else
        CELEG_REQUIRE(false, "gated_head_norm: unknown dtype code %d", act_dtype);
    return check_launch("gated_head_norm");
}

// One token per request (row i of ``proj`` is request i's token, its slot span_slot[i]): everything between the
// two projections of a matrix-state mixer in one launch. mode 0 (delta): the convolved channels [q | k | v] are
// the first ``channels`` columns of a row, bias0 = A_log, bias1 = dt_bias, the output gate is SiLU; the carried
// inputs are moved on by a second launch. mode 1 (mLSTM): bias0 / bias1 = the gates' biases, the gate is a sigmoid.
// mode 2 (retention): bias0 = the heads' decays, the output gate is SiLU, norm_w may be null (no weight).
static int recurrent_decode_launch(int mode, const float* proj, int stride, int q_off, int k_off, int v_off,
                                   int gate_off, int g0_off, int g1_off, const float* conv_kernel, float* carried,
                                   int taps, int channels, const float* bias0, const float* bias1, float cap,
                                   const float* norm_w, int norm_per_head, float eps, float unit_eps, float* state,
                                   long long slot_stride, const int* span_begin, const int* span_slot, int tokens,
                                   int heads, int kv_heads, int dim, int vdim, float q_scale, void* out,
                                   int act_dtype, int input_act, float* raw_out, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0,
                  "recurrent_decode: invalid sizes tokens=%d heads=%d kv_heads=%d dim=%d vdim=%d", tokens, heads,
                  kv_heads, dim, vdim);
    CELEG_REQUIRE(mode == kScanDelta || mode == kScanMlstm || mode == kScanRetention, "recurrent_decode: unknown mode %d", mode);
    CELEG_REQUIRE(mode != kScanDelta || (taps >= 1 && taps <= 16 && conv_kernel && (taps == 1 || carried)),
                  "recurrent_decode: the delta rule needs its kernel of 1 to 16 taps and the carried inputs");
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "recurrent_decode: unknown dtype code %d", act_dtype);
    CELEG_REQUIRE(tokens <= 65535, "recurrent_decode: %d tokens exceed one launch", tokens);
    constexpr int kDecodeStepThreads = 256;
    const size_t smem = (size_t)(2 * dim + vdim + 2 * kDecodeStepThreads) * sizeof(float);
    CELEG_REQUIRE(smem <= 40 * 1024, "recurrent_decode: head sizes %d and %d exceed a block's shared memory", dim, vdim);
    if (tokens == 0) return 0;
    const DecodeStepParams p = {proj, stride, q_off, k_off, v_off, gate_off, g0_off, g1_off, conv_kernel, carried, taps,
                                channels, bias0, bias1, cap, norm_w, norm_per_head, eps, unit_eps, state, slot_stride,
                                span_slot, heads, kv_heads, dim, vdim, q_scale, out, input_act, raw_out};
    dim3 grid(heads, tokens);
    if (mode == kScanDelta) {
        if (act_dtype == kFloat32)
            launch_chained(recurrent_decode_kernel<kScanDelta, float>, grid, kDecodeStepThreads, smem, stream, p);
        else
            launch_chained(recurrent_decode_kernel<kScanDelta, __nv_bfloat16>, grid, kDecodeStepThreads, smem, stream, p);
        int status = check_launch("recurrent_decode");
        if (status != 0 || taps == 1) return status;
        const long long units = (long long)tokens * channels;
        launch_chained(carried_inputs_update_kernel, (unsigned)((units + 127) / 128), 128, 0, stream, proj, stride,
                       carried, slot_stride, span_begin, span_slot, tokens, channels, taps);
        return check_launch("carried_inputs_update");
    }
    if (mode == kScanRetention) {
        if (act_dtype == kFloat32)
            launch_chained(recurrent_decode_kernel<kScanRetention, float>, grid, kDecodeStepThreads, smem, stream, p);
        else
            launch_chained(recurrent_decode_kernel<kScanRetention, __nv_bfloat16>, grid, kDecodeStepThreads, smem, stream, p);
        return check_launch("recurrent_decode");
    }
    if (act_dtype == kFloat32)
        launch_chained(recurrent_decode_kernel<kScanMlstm, float>, grid, kDecodeStepThreads, smem, stream, p);
    else
        launch_chained(recurrent_decode_kernel<kScanMlstm, __nv_bfloat16>, grid, kDecodeStepThreads, smem, stream, p);
    return check_launch("recurrent_decode");
}

CELEG_API int celeg_recurrent_decode(int mode, const float* proj, int stride, int q_off, int k_off, int v_off,
                                     int gate_off, int g0_off, int g1_off, const float* conv_kernel, float* carried,
                                     int taps, int channels, const float* bias0, const float* bias1, float cap,
                                     const float* norm_w, int norm_per_head, float eps, float unit_eps, float* state,
                                     long long slot_stride, const int* span_begin, const int* span_slot, int tokens,
                                     int heads, int kv_heads, int dim, int vdim, float q_scale, void* out,
                                     int act_dtype, cudaStream_t stream) {
    return recurrent_decode_launch(mode, proj, stride, q_off, k_off, v_off, gate_off, g0_off, g1_off, conv_kernel, carried,
                                   taps, channels, bias0, bias1, cap, norm_w, norm_per_head, eps, unit_eps, state,
                                   slot_stride, span_begin, span_slot, tokens, heads, kv_heads, dim, vdim, q_scale, out,
                                   act_dtype, -1, nullptr, stream);
}

// The retention's decoding step with an activation of q, k and v as they are read (input_act: a code of activate(), or
// -1) and the read-outs left as they are in raw_out (float32 [tokens, heads * vdim]): for a mixer whose norm runs over
// all heads together, which no block of this launch sees.
CELEG_API int celeg_retention_decode_raw(const float* proj, int stride, int q_off, int k_off, int v_off,
                                         const float* decay, float* state, long long slot_stride, const int* span_slot,
                                         int tokens, int heads, int dim, int vdim, float q_scale, int input_act,
                                         float* raw_out, cudaStream_t stream) {
    CELEG_REQUIRE(raw_out != nullptr && input_act >= -1 && input_act <= 3, "retention_decode_raw: no output or activation %d",
                  input_act);
    return recurrent_decode_launch(kScanRetention, proj, stride, q_off, k_off, v_off, 0, 0, 0, nullptr, nullptr, 0, 0, decay,
                                   decay, 0.0f, nullptr, 0, 1.0f, 0.0f, state, slot_stride, nullptr, span_slot, tokens,
                                   heads, heads, dim, vdim, q_scale, raw_out, kFloat32, input_act, raw_out, stream);
}

// Retention over the step's spans in segments of `segment` tokens (a multiple of 64). Scratch: floats
// [2 * max_segments * heads * dim * vdim] (the segments' own states, then the states at their starts), ints
// [max_segments + spans + 2] (segment starts, the spans' first segments), with max_segments >= tokens / segment +
// spans; identity: the numbers 0 .. max_segments - 1. decay: [heads]. Same result as mode 2 of celeg_recurrent_scan
// but for rounding.
CELEG_API int celeg_retention_segmented(const float* q, int q_stride, const float* k, int k_stride, const float* v,
                                        int v_stride, const float* decay, float* out, float* state, long long slot_stride,
                                        const int* span_begin, const int* span_slot, int spans, int tokens, int heads,
                                        int dim, int vdim, float q_scale, int segment, int max_segments,
                                        float* float_scratch, int* int_scratch, const int* identity,
                                        cudaStream_t stream) {
    CELEG_REQUIRE(spans >= 0 && tokens >= 0 && heads > 0 && dim > 0 && vdim > 0 && segment >= 64 && segment % 64 == 0,
                  "retention_segmented: invalid sizes spans=%d tokens=%d heads=%d dim=%d vdim=%d segment=%d", spans, tokens,
                  heads, dim, vdim, segment);
    CELEG_REQUIRE(dim <= kScanMaxDim, "retention_segmented: a key size of %d exceeds %d", dim, kScanMaxDim);
    CELEG_REQUIRE(max_segments >= tokens / segment + spans && max_segments <= 65535 && spans <= 65535 && heads <= 65535,
                  "retention_segmented: %d segments do not hold %d tokens in %d spans (or exceed one launch)", max_segments,
                  tokens, spans);
    if (spans == 0 || tokens == 0) return 0;
    const long long elements = (long long)heads * dim * vdim;
    float* local = float_scratch;
    float* carried = float_scratch + (size_t)max_segments * elements;
    int* seg_begin = int_scratch;                          // [max_segments + 1]
    int* span_first = int_scratch + max_segments + 1;      // [spans + 1]
    cudaMemsetAsync(local, 0, (size_t)max_segments * elements * sizeof(float), stream);
    launch_chained(retention_plan_kernel, 1, 32, 0, stream, span_begin, spans, segment, max_segments, seg_begin, span_first);
    int status = check_launch("retention_plan");
    if (status != 0) return status;
    const int vector_copies = dim % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && (((size_t)q | (size_t)k) & 15) == 0;
    const ScanParams p = {q, k, v, q_stride, k_stride, v_stride, decay, out, local, elements, seg_begin, identity,
                          heads, heads, dim, vdim, q_scale, vector_copies};
    status = launch_wide_scan(p, max_segments, stream);
    if (status != 0) return status;
    dim3 carry_grid((unsigned)((elements + 255) / 256), spans);
    retention_carry_kernel<<<carry_grid, 256, 0, stream>>>(state, slot_stride, span_slot, span_first, seg_begin, local,
                                                            carried, decay, (int)elements, dim * vdim);
    status = check_launch("retention_carry");
    if (status != 0) return status;
    const int pieces = segment / 64;
    dim3 add_grid((vdim + 63) / 64, heads, max_segments * pieces);
    CELEG_REQUIRE((long long)max_segments * pieces <= 65535, "retention_segmented: %d segments of %d pieces exceed one launch",
                  max_segments, pieces);
    retention_add_carried_kernel<<<add_grid, 256, 0, stream>>>(q, q_stride, carried, seg_begin, decay, out, heads, dim, vdim,
                                                                pieces);
    return check_launch("retention_add_carried");
}
