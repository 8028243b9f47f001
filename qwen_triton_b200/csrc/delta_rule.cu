// A recurrent mixer: the gated delta rule with one decay per head and key channel, and what surrounds it.
//
// Per head, with a state S [dim, vdim] of float that is carried from token to token of a sequence:
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// (o_t is read after token t has been written).  q and k come from kv heads (head h reads kv head h / (heads / kv_heads)),
// are unit vectors per head (q also times dim^-1/2), and q, k, v have passed a short causal convolution per channel and
// SiLU.  Everything here is float whatever the model's element type: the projections before it hand over float sums.
//
// Kernels, in the order of a step:
//   delta_prepare_kernel   convolution (its first taps - 1 inputs from the sequence's kept inputs or from zeros), SiLU, unit
//                          norms, beta = sigmoid(.)
//   conv_keep_kernel       the last taps - 1 raw inputs of every sequence, kept for its next step
//   lowrank_kernel         y = f(W2 (x) + bias) for a projection through a few columns (x is a slice of the first
//                          projection's output): f = -exp(rate_h) softplus(.), the logarithm of the decays, or sigmoid for a gate
//   delta_step_kernel      the recurrence token by token (steps of few tokens per sequence: a state is read and written once
//                          per step anyway, and the kernel is laid out for those bytes); delta_scan_kernel is an older
//                          form of it (QT_B200_DELTA_STEP=0), a column's rows over 8 lanes
//   delta_chunk_prepare_kernel, delta_chunk_scan_kernel
//                          the same recurrence in chunks of 16 tokens for longer steps (see there)
//   gated_head_norm_kernel o / rms(o) * w * gate per head, into the element type of the output projection's input
#include "common.cuh"

#include <math.h>

using namespace qt;

constexpr int MAX_TAPS = 16;

struct PrepareParams {
    const float* proj; int n_splits; size_t split_stride; int proj_cols;    // [splits, T, proj_cols]; columns: q | k | v | beta | ...
    const float* taps;                // [channels, n_taps], the last column is the current token's
    const float* kept;                // [slots + 1, n_taps - 1, channels]: raw inputs of the positions just before the step
    const int* token_seq; const int* token_pos; const int* seq_start; const int* seq_past; const int* slots;
    float* q; float* k; float* v; float* beta;      // [T, kv_heads, dim] x 2, [T, heads, vdim], [T, heads]
    int n_tokens, heads, kv_heads, dim, vdim, n_taps;
    float unit_eps;
};

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }

// The sum of split-K partial sums in their order, eight loads in flight at a time.
__device__ __forceinline__ float sum_splits(const float* __restrict__ base, size_t index, int n_splits, size_t split_stride) {
    if (n_splits == 1) return base[index];
    float acc = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = s0 + j < n_splits ? base[index + (size_t)(s0 + j) * split_stride] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += v[j];
    }
    return acc;
}
__device__ __forceinline__ float softplusf(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// One warp per (token, item): items 0 .. kv_heads - 1 are the q heads, the next kv_heads the k heads, the next `heads`
// the v heads, the last one all betas of the token.
__global__ void __launch_bounds__(128) delta_prepare_kernel(const PrepareParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items = 2 * p.kv_heads + p.heads + 1;
    const long long index = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (index >= (long long)p.n_tokens * items) return;
    const int t = (int)(index / items), item = (int)(index % items);
    const size_t row = (size_t)t * p.proj_cols;
    const int channels = 2 * p.kv_heads * p.dim + p.heads * p.vdim;
    if (item == items - 1) {
        for (int h = lane; h < p.heads; h += 32)
            p.beta[(size_t)t * p.heads + h] = sigmoidf(sum_splits(p.proj, row + channels + h, p.n_splits, p.split_stride));
        return;
    }
    const int seq = p.token_seq[t];
    const int local = p.token_pos[t] - p.seq_past[seq];          // tokens of this sequence that the step has run before this one
    const float* kept = p.kept + (size_t)p.slots[seq] * (p.n_taps - 1) * channels;
    const bool is_q = item < p.kv_heads, is_k = !is_q && item < 2 * p.kv_heads;
    const int width = (is_q || is_k) ? p.dim : p.vdim;
    const int c0 = is_q ? item * p.dim : is_k ? p.kv_heads * p.dim + (item - p.kv_heads) * p.dim
                                              : 2 * p.kv_heads * p.dim + (item - 2 * p.kv_heads) * p.vdim;
    float* out = is_q ? p.q + ((size_t)t * p.kv_heads + item) * p.dim
               : is_k ? p.k + ((size_t)t * p.kv_heads + item - p.kv_heads) * p.dim
                      : p.v + ((size_t)t * p.heads + item - 2 * p.kv_heads) * p.vdim;
    float sq = 0.f;
    const float* __restrict__ proj = p.proj;
    const float* __restrict__ taps = p.taps;
    for (int i = lane; i < width; i += 32) {
        const int c = c0 + i;
        float acc = 0.f;
        for (int back0 = 0; back0 < p.n_taps; back0 += 4) {           // four taps at a time: their loads go out together
            float x[4], w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int back = back0 + j;
                x[j] = w[j] = 0.f;
                if (back < p.n_taps) {
                    w[j] = taps[(size_t)c * p.n_taps + p.n_taps - 1 - back];
                    if (back <= local) x[j] = sum_splits(proj, row - (size_t)back * p.proj_cols + c, p.n_splits, p.split_stride);
                    else x[j] = kept[(size_t)(p.n_taps - 1 - (back - local)) * channels + c];
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) acc += w[j] * x[j];
        }
        const float y = acc / (1.f + expf(-acc));
        out[i] = y;
        sq += y * y;
    }
    if (is_q || is_k) {
        const float inv = rsqrtf(warp_sum(sq) + p.unit_eps) * (is_q ? rsqrtf((float)p.dim) : 1.f);
        __syncwarp();
        for (int i = lane; i < width; i += 32) out[i] *= inv;
    }
}

// kept[slot] <- the raw inputs of the sequence's last n_taps - 1 positions after this step.  One thread per
// (sequence, channel): it reads what it needs of the old rows before it writes.
__global__ void conv_keep_kernel(const float* __restrict__ proj, int n_splits, size_t split_stride, int proj_cols,
                                 float* __restrict__ kept, const int* __restrict__ seq_start, const int* __restrict__ slots,
                                 int n_seqs, int channels, int n_taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int row0 = seq_start[seq], count = seq_start[seq + 1] - row0;
    float* mine = kept + (size_t)slots[seq] * (n_taps - 1) * channels + c;
    float value[MAX_TAPS];
    const int rows = n_taps - 1;
    for (int j = 0; j < rows; ++j) {
        const int from = count - rows + j;                       // index among the step's tokens; negative: an older position
        value[j] = from >= 0 ? sum_splits(proj, (size_t)(row0 + from) * proj_cols + c, n_splits, split_stride)
                             : mine[(size_t)(rows + from) * channels];
    }
    for (int j = 0; j < rows; ++j) mine[(size_t)j * channels] = value[j];
}

// out[t, n] = f(sum_r w[r, n] x[t, r] + bias[n]) for a tile of LR_TOKENS tokens and 256 outputs per block.
constexpr int LR_TOKENS = 16;
constexpr int LR_DECAY = 0, LR_SIGMOID = 1;

template <int MODE>
__global__ void __launch_bounds__(256) lowrank_kernel(const float* __restrict__ proj, int n_splits, size_t split_stride, int proj_cols,
                                                      int x_offset, int rank, const float* __restrict__ w, const float* __restrict__ bias,
                                                      const float* __restrict__ rate_log, int per_rate, float* __restrict__ out,
                                                      int n_tokens, int n_out) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float xs[];                   // [rank][LR_TOKENS]: a column's 16 tokens side by side
    const int t0 = blockIdx.y * LR_TOKENS;
    const int count = min(LR_TOKENS, n_tokens - t0);
    for (int i = threadIdx.x; i < LR_TOKENS * rank; i += blockDim.x) {
        const int tt = i / rank, r = i % rank;
        xs[r * LR_TOKENS + tt] = tt < count ? sum_splits(proj, (size_t)(t0 + tt) * proj_cols + x_offset + r, n_splits, split_stride) : 0.f;
    }
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= n_out) return;
    float acc[LR_TOKENS];
#pragma unroll
    for (int tt = 0; tt < LR_TOKENS; ++tt) acc[tt] = 0.f;
    for (int r0 = 0; r0 < rank; r0 += 8) {                            // eight weights at a time: their loads go out together
        float wv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) wv[j] = r0 + j < rank ? w[(size_t)(r0 + j) * n_out + n] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (r0 + j < rank) {
                const float4* x4 = reinterpret_cast<const float4*>(xs + (r0 + j) * LR_TOKENS);
#pragma unroll
                for (int q = 0; q < LR_TOKENS / 4; ++q) {
                    const float4 x = x4[q];
                    acc[4 * q] += wv[j] * x.x; acc[4 * q + 1] += wv[j] * x.y; acc[4 * q + 2] += wv[j] * x.z; acc[4 * q + 3] += wv[j] * x.w;
                }
            }
        }
    }
    const float b = bias ? bias[n] : 0.f;
    const float rate = MODE == LR_DECAY ? expf(rate_log[n / per_rate]) : 0.f;
#pragma unroll
    for (int tt = 0; tt < LR_TOKENS; ++tt) {
        if (tt >= count) break;
        const float z = acc[tt] + b;
        out[(size_t)(t0 + tt) * n_out + n] = MODE == LR_DECAY ? -rate * softplusf(z) : sigmoidf(z);     // the decay's logarithm
    }
}

// The same for a step of few tokens (up to 16 tiles of them): 64 outputs per block, so that many SMs get one, and the
// columns cut into four ranges, one per 64 threads, whose sums meet in shared memory.
template <int MODE>
__global__ void __launch_bounds__(256) lowrank_few_kernel(const float* __restrict__ proj, int n_splits, size_t split_stride, int proj_cols,
                                                          int x_offset, int rank, const float* __restrict__ w, const float* __restrict__ bias,
                                                          const float* __restrict__ rate_log, int per_rate, float* __restrict__ out,
                                                          int n_tokens, int n_out) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];                                 // [LR_TOKENS][rank], then [4][LR_TOKENS][64] partial sums
    float* part = xs + LR_TOKENS * rank;
    const int t0 = blockIdx.y * LR_TOKENS;
    n_tokens = min(LR_TOKENS, n_tokens - t0);                     // of this tile
    out += (size_t)t0 * n_out;
    for (int i = threadIdx.x; i < LR_TOKENS * rank; i += blockDim.x) {
        const int tt = i / rank, r = i % rank;
        xs[i] = tt < n_tokens ? sum_splits(proj, (size_t)(t0 + tt) * proj_cols + x_offset + r, n_splits, split_stride) : 0.f;
    }
    __syncthreads();
    const int local = threadIdx.x & 63, slice = threadIdx.x >> 6;
    const int n = blockIdx.x * 64 + local;
    const int per = (rank + 3) / 4, r_begin = slice * per, r_end = min(rank, r_begin + per);
    float acc[LR_TOKENS];
#pragma unroll
    for (int tt = 0; tt < LR_TOKENS; ++tt) acc[tt] = 0.f;
    if (n < n_out) {
        for (int r0 = r_begin; r0 < r_end; r0 += 8) {
            float wv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[j] = r0 + j < r_end ? w[(size_t)(r0 + j) * n_out + n] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (r0 + j < r_end) {
#pragma unroll
                    for (int tt = 0; tt < LR_TOKENS; ++tt) acc[tt] += wv[j] * xs[tt * rank + r0 + j];
                }
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < LR_TOKENS; ++tt) part[(slice * LR_TOKENS + tt) * 64 + local] = acc[tt];
    __syncthreads();
    if (n >= n_out) return;
    const float b = bias ? bias[n] : 0.f;
    const float rate = MODE == LR_DECAY ? expf(rate_log[n / per_rate]) : 0.f;
    for (int tt = slice; tt < n_tokens; tt += 4) {                 // the four ranges' sums in their order
        const float z = part[(0 * LR_TOKENS + tt) * 64 + local] + part[(1 * LR_TOKENS + tt) * 64 + local] +
                        part[(2 * LR_TOKENS + tt) * 64 + local] + part[(3 * LR_TOKENS + tt) * 64 + local] + b;
        out[(size_t)tt * n_out + n] = MODE == LR_DECAY ? -rate * softplusf(z) : sigmoidf(z);
    }
}

// ----------------------------------------------------------------------------- the recurrence
// grid (column blocks, heads, sequences).  A block of 256 threads owns SCAN_COLS = 32 columns of one head's state; a
// column belongs to 8 neighbouring lanes, lane s of them holding rows s, s + 8, ... (R of them) in registers.  The
// tokens' q, k and decays (shared by the block), and the block's v columns and beta, pass through shared memory in chunks
// of SCAN_CHUNK tokens, the next chunk fetched (cp.async) while this one is worked on.
constexpr int SCAN_COLS = 32;
constexpr int SCAN_LANES = 8;
constexpr int SCAN_CHUNK = 16;

struct ScanParams {
    const float* q; const float* k; const float* v; const float* beta; const float* decay;      // decay: logarithms, [T, heads, dim]
    float* state;                 // [slots + 1, heads, dim, vdim]
    float* out;                   // [T, heads, vdim]
    const int* seq_start; const int* slots;
    int heads, kv_heads, dim, vdim;
};

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int R>
__global__ void __launch_bounds__(SCAN_COLS * SCAN_LANES) delta_scan_kernel(const ScanParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int dim = p.dim, vdim = p.vdim;
    const int per_token = 3 * dim + SCAN_COLS + 1;                 // q, k, decay, the block's v columns, beta
    float* buffers[2] = {sm, sm + SCAN_CHUNK * per_token};
    const int head = blockIdx.y, seq = blockIdx.z;
    const int kvh = head / (p.heads / p.kv_heads);
    const int col = threadIdx.x / SCAN_LANES, sub = threadIdx.x % SCAN_LANES;
    const int j = blockIdx.x * SCAN_COLS + col;
    const bool live = j < vdim;
    const int row0 = p.seq_start[seq], count = p.seq_start[seq + 1] - row0;
    float* state = p.state + ((size_t)p.slots[seq] * p.heads + head) * dim * vdim;

    float s[R];
#pragma unroll
    for (int m = 0; m < R; ++m) {
        const int i = sub + SCAN_LANES * m;
        s[m] = (live && i < dim) ? state[(size_t)i * vdim + j] : 0.f;
    }
    auto fetch = [&](int chunk, float* buf) {
        const int first = chunk * SCAN_CHUNK, n = min(SCAN_CHUNK, count - first);
        for (int e = threadIdx.x; e < n * per_token; e += blockDim.x) {
            const int tt = e / per_token, c = e % per_token;
            const size_t t = (size_t)(row0 + first + tt);
            const float* src;
            if (c < dim) src = p.q + (t * p.kv_heads + kvh) * dim + c;
            else if (c < 2 * dim) src = p.k + (t * p.kv_heads + kvh) * dim + (c - dim);
            else if (c < 3 * dim) src = p.decay + (t * p.heads + head) * dim + (c - 2 * dim);
            else if (c < 3 * dim + SCAN_COLS) {
                const int jj = blockIdx.x * SCAN_COLS + (c - 3 * dim);
                src = p.v + (t * p.heads + head) * vdim + (jj < vdim ? jj : vdim - 1);
            } else src = p.beta + t * p.heads + head;
            cp_async4(buf + e, src);
        }
        cp_async_commit();
    };
    const int chunks = (count + SCAN_CHUNK - 1) / SCAN_CHUNK;
    if (chunks > 0) fetch(0, buffers[0]);
    for (int chunk = 0; chunk < chunks; ++chunk) {
        cp_async_wait_all();
        __syncthreads();                                           // this chunk has landed; everyone is done with the other buffer
        if (chunk + 1 < chunks) fetch(chunk + 1, buffers[(chunk + 1) & 1]);
        const float* buf = buffers[chunk & 1];
        const int n = min(SCAN_CHUNK, count - chunk * SCAN_CHUNK);
        for (int tt = 0; tt < n; ++tt) {
            const float* q = buf + tt * per_token;
            const float* k = q + dim;
            const float* g = k + dim;
            const float vj = q[3 * dim + col], beta = q[3 * dim + SCAN_COLS];
            float kk[R];
            float pred = 0.f;
#pragma unroll
            for (int m = 0; m < R; ++m) {
                const int i = sub + SCAN_LANES * m;
                const bool in = i < dim;
                kk[m] = in ? k[i] : 0.f;
                s[m] *= in ? expf(g[i]) : 1.f;                      // `decay` holds logarithms
                pred += s[m] * kk[m];
            }
            pred += __shfl_xor_sync(0xffffffffu, pred, 1);
            pred += __shfl_xor_sync(0xffffffffu, pred, 2);
            pred += __shfl_xor_sync(0xffffffffu, pred, 4);
            const float u = beta * (vj - pred);
            float o = 0.f;
#pragma unroll
            for (int m = 0; m < R; ++m) {
                const int i = sub + SCAN_LANES * m;
                s[m] += kk[m] * u;
                o += s[m] * (i < dim ? q[i] : 0.f);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (sub == 0 && live) p.out[((size_t)(row0 + chunk * SCAN_CHUNK + tt) * p.heads + head) * vdim + j] = o;
        }
    }
#pragma unroll
    for (int m = 0; m < R; ++m) {
        const int i = sub + SCAN_LANES * m;
        if (live && i < dim) state[(size_t)i * vdim + j] = s[m];
    }
}

// ----------------------------------------------------------------------------- the recurrence in chunks
// Within a chunk of CH tokens that starts from the state S0, with L_t the sum of the decays' logarithms up to token t
// of the chunk (per key channel), the recurrence unrolls to
//     u_t = beta_t (v_t - S0^T (e^{L_t} k_t) - sum_{s<t} A[t,s] u_s),      A[t,s] = sum_c k_t[c] k_s[c] e^{L_t[c] - L_s[c]}
//     o_t = S0^T (e^{L_t} q_t) + sum_{s<=t} B[t,s] u_s,                    B[t,s] = sum_c q_t[c] k_s[c] e^{L_t[c] - L_s[c]}
//     S   = diag(e^{L_last}) S0 + sum_s (e^{L_last - L_s} k_s) u_s^T
// Every exponent is a sum of logarithms of decays over a range of tokens, so it is <= 0: nothing is divided by a decay.
// What does not depend on the state (the scaled keys and queries and the two triangles) is made for all chunks of all
// heads at once by delta_chunk_prepare_kernel; delta_chunk_scan_kernel then walks the chunks of a sequence with the
// state's columns in registers, and its work per chunk has no chain from token to token but the small triangular
// solve.  All float; the result differs from the token-by-token kernel by rounding only.
constexpr int CH = 16;
constexpr int AB = 2 * CH + 4;      // floats of a token's row of `ab`: its columns of the two triangles, beta, padding to 16 bytes

struct ChunkParams {
    const float* q; const float* k; const float* log_decay;      // [T, kv_heads, dim] x 2, [T, heads, dim]
    float* kt; float* qt; float* kb; float* gc;                    // [T, heads, dim]: e^{L_t} k_t, e^{L_t} q_t, e^{L_last - L_t} k_t; e^{L_last} in a chunk's first row
    const float* beta;                                             // [T, heads]
    float* ab;                                                     // [T, heads, AB]: beta_s at [2 CH], and for token s, A[t, s] for every t of its chunk (0 unless s < t), then B[t, s] (0 unless s <= t)
    const int* seq_start;
    int heads, kv_heads, dim;
};

// grid (chunks of the longest sequence, heads, sequences), 128 threads.
__global__ void __launch_bounds__(128) delta_chunk_prepare_kernel(const ChunkParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int dim = p.dim, head = blockIdx.y, seq = blockIdx.z;
    const int kvh = head / (p.heads / p.kv_heads);
    const int row0 = p.seq_start[seq], count = p.seq_start[seq + 1] - row0;
    const int first = blockIdx.x * CH;
    if (first >= count) return;
    const int n = min(CH, count - first);
    float* qs = sm;                       // [CH][dim]
    float* ks = qs + CH * dim;            // [CH][dim]
    float* ls = ks + CH * dim;            // [CH][dim] running sums of the logarithms
    for (int e = threadIdx.x; e < CH * dim; e += blockDim.x) {
        const int tt = e / dim, c = e % dim;
        const size_t t = (size_t)(row0 + first + tt);
        const bool in = tt < n;
        qs[e] = in ? p.q[(t * p.kv_heads + kvh) * dim + c] : 0.f;
        ks[e] = in ? p.k[(t * p.kv_heads + kvh) * dim + c] : 0.f;
        ls[e] = in ? p.log_decay[(t * p.heads + head) * dim + c] : 0.f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float run = 0.f;
        for (int tt = 0; tt < CH; ++tt) { run += ls[tt * dim + c]; ls[tt * dim + c] = run; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * dim; e += blockDim.x) {
        const int tt = e / dim, c = e % dim;
        const size_t at = ((size_t)(row0 + first + tt) * p.heads + head) * dim + c;
        const float grow = expf(ls[e]), rest = expf(ls[(n - 1) * dim + c] - ls[e]);
        p.kt[at] = grow * ks[e];
        p.qt[at] = grow * qs[e];
        p.kb[at] = rest * ks[e];
        if (tt == 0) p.gc[at] = expf(ls[(n - 1) * dim + c]);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int pair = warp; pair < CH * CH; pair += 4) {
        const int s = pair / CH, t = pair % CH;
        if (s >= n) break;
        float a = 0.f, b = 0.f;
        if (s <= t && t < n) {
            for (int c = lane; c < dim; c += 32) {
                const float w = ks[s * dim + c] * expf(ls[t * dim + c] - ls[s * dim + c]);
                a += ks[t * dim + c] * w;
                b += qs[t * dim + c] * w;
            }
            a = warp_sum(a);
            b = warp_sum(b);
        }
        if (lane == 0) {
            float* row = p.ab + ((size_t)(row0 + first + s) * p.heads + head) * AB;
            row[t] = s < t ? a : 0.f;
            row[CH + t] = b;
            if (t == 0) row[2 * CH] = p.beta[(size_t)(row0 + first + s) * p.heads + head];
        }
    }
}

struct ChunkScanParams {
    const float* kt; const float* qt; const float* kb; const float* gc; const float* ab;
    const float* v; const float* beta;
    float* state; float* out;
    const int* seq_start; const int* slots;
    int heads, dim, vdim;
};

// grid (column blocks, heads, sequences); threads as in delta_scan_kernel: a column of the state belongs to 8 neighbouring
// lanes, lane s of them holding rows s, s + 8, ...
template <int R>
__global__ void __launch_bounds__(SCAN_COLS * SCAN_LANES) delta_chunk_scan_kernel(const ChunkScanParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int dim = p.dim, vdim = p.vdim;
    const int per_token = 3 * dim + 2 * CH + SCAN_COLS + 1;       // kt, qt, kb rows, the A and B rows, the block's v columns, beta
    const int per_chunk = CH * per_token + dim;                   // and the chunk's whole decay
    float* buffers[2] = {sm, sm + per_chunk};
    const int head = blockIdx.y, seq = blockIdx.z;
    const int col = threadIdx.x / SCAN_LANES, sub = threadIdx.x % SCAN_LANES;
    const int j = blockIdx.x * SCAN_COLS + col;
    const bool live = j < vdim;
    const int row0 = p.seq_start[seq], count = p.seq_start[seq + 1] - row0;
    float* state = p.state + ((size_t)p.slots[seq] * p.heads + head) * dim * vdim;

    float s[R];
#pragma unroll
    for (int m = 0; m < R; ++m) {
        const int i = sub + SCAN_LANES * m;
        s[m] = (live && i < dim) ? state[(size_t)i * vdim + j] : 0.f;
    }
    auto fetch = [&](int chunk, float* buf) {
        const int first = chunk * CH, n = min(CH, count - first);
        for (int e = threadIdx.x; e < n * per_token + dim; e += blockDim.x) {
            const float* src;
            float* dst;
            if (e < n * per_token) {
                const int tt = e / per_token, c = e % per_token;
                const size_t at = (size_t)(row0 + first + tt) * p.heads + head;
                if (c < dim) src = p.kt + at * dim + c;
                else if (c < 2 * dim) src = p.qt + at * dim + (c - dim);
                else if (c < 3 * dim) src = p.kb + at * dim + (c - 2 * dim);
                else if (c < 3 * dim + 2 * CH) src = p.ab + at * AB + (c - 3 * dim);
                else if (c < 3 * dim + 2 * CH + SCAN_COLS) {
                    const int jj = blockIdx.x * SCAN_COLS + (c - 3 * dim - 2 * CH);
                    src = p.v + at * vdim + (jj < vdim ? jj : vdim - 1);
                } else src = p.beta + at;
                dst = buf + e;
            } else {
                src = p.gc + ((size_t)(row0 + first) * p.heads + head) * dim + (e - n * per_token);
                dst = buf + CH * per_token + (e - n * per_token);
            }
            cp_async4(dst, src);
        }
        cp_async_commit();
    };
    const int chunks = (count + CH - 1) / CH;
    if (chunks > 0) fetch(0, buffers[0]);
    for (int chunk = 0; chunk < chunks; ++chunk) {
        cp_async_wait_all();
        __syncthreads();
        if (chunk + 1 < chunks) fetch(chunk + 1, buffers[(chunk + 1) & 1]);
        const float* buf = buffers[chunk & 1];
        const int n = min(CH, count - chunk * CH);
        // what the state holds for every token of the chunk: S0^T (e^L k_t) and S0^T (e^L q_t), summed over the 8 lanes of the column
        float pred[CH], read[CH];
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
            float a = 0.f, b = 0.f;
            if (tt < n) {
                const float* kt = buf + tt * per_token;
                const float* qt = kt + dim;
#pragma unroll
                for (int m = 0; m < R; ++m) {
                    const int i = sub + SCAN_LANES * m;
                    if (i < dim) { a += kt[i] * s[m]; b += qt[i] * s[m]; }
                }
            }
            pred[tt] = a;
            read[tt] = b;
        }
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
            pred[tt] += __shfl_xor_sync(0xffffffffu, pred[tt], 1);
            read[tt] += __shfl_xor_sync(0xffffffffu, read[tt], 1);
            pred[tt] += __shfl_xor_sync(0xffffffffu, pred[tt], 2);
            read[tt] += __shfl_xor_sync(0xffffffffu, read[tt], 2);
            pred[tt] += __shfl_xor_sync(0xffffffffu, pred[tt], 4);
            read[tt] += __shfl_xor_sync(0xffffffffu, read[tt], 4);
        }
        // the triangular solve, the same in each of the column's lanes; pred[t] turns into u_t
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
            if (tt < n) {
                const float* row = buf + tt * per_token + 3 * dim;            // the token's columns of A and B, v columns, beta
                const float u = row[2 * CH + SCAN_COLS] * (row[2 * CH + col] - pred[tt]);
                pred[tt] = u;
#pragma unroll
                for (int later = tt + 1; later < CH; ++later)
                    if (later < n) pred[later] += row[later] * u;
#pragma unroll
                for (int later = tt; later < CH; ++later)
                    if (later < n) read[later] += row[CH + later] * u;
            }
        }
        if (sub == 0 && live) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt)
                if (tt < n) p.out[((size_t)(row0 + chunk * CH + tt) * p.heads + head) * vdim + j] = read[tt];
        }
        // the state behind the chunk
        const float* gc = buf + CH * per_token;
#pragma unroll
        for (int m = 0; m < R; ++m) {
            const int i = sub + SCAN_LANES * m;
            if (i < dim) {
                float acc = gc[i] * s[m];
#pragma unroll
                for (int tt = 0; tt < CH; ++tt)
                    if (tt < n) acc += buf[tt * per_token + 2 * dim + i] * pred[tt];
                s[m] = acc;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < R; ++m) {
        const int i = sub + SCAN_LANES * m;
        if (live && i < dim) state[(size_t)i * vdim + j] = s[m];
    }
}

// The same walk for the usual sizes (dim a multiple of 64 up to 256, vdim a multiple of 16), written for few instructions:
// a column of the state belongs to CH = 16 neighbouring lanes, lane l of them holding the rows 4 (l + 16 q) + e
// (q < RQ, e < 4: 16-byte pieces that the 16 lanes read side by side) and owning the scalars of the chunk's token l.
// The per-token sums over the state's rows are reduced so that token l's sum lands in lane l (15 exchanges instead of
// 64), the triangular solve passes each u_t on by one shuffle, and chunk data arrives by 16-byte copies; a chunk's
// missing tokens are zeros, which change nothing.  grid (vdim / 16, heads, sequences), 256 threads.
constexpr int FAST_COLS = 16;

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// LPC lanes per column: 16 as described, or 32 (a warp per column, dim a multiple of 128: twice the warps, each with half
// the rows; lanes l and l + 16 then both carry token l's scalars).
template <int LPC, int RQ>
__global__ void __launch_bounds__(FAST_COLS * LPC) delta_chunk_scan_fast_kernel(const ChunkScanParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int DIM = 4 * LPC * RQ;
    constexpr int PER_TOKEN = 3 * DIM + AB + FAST_COLS;           // kt, qt, kb rows, the token's row of `ab` (with beta), v columns
    constexpr int PER_CHUNK = CH * PER_TOKEN + DIM;
    float* buffers[2] = {sm, sm + PER_CHUNK};
    const int vdim = p.vdim, head = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x & 31, row_lane = threadIdx.x & (LPC - 1), l = threadIdx.x & 15, col = threadIdx.x / LPC;
    const int j = blockIdx.x * FAST_COLS + col;
    const int row0 = p.seq_start[seq], count = p.seq_start[seq + 1] - row0;
    float* state = p.state + ((size_t)p.slots[seq] * p.heads + head) * DIM * vdim;

    float s[RQ][4];
#pragma unroll
    for (int q = 0; q < RQ; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[q][e] = state[(size_t)(4 * (row_lane + LPC * q) + e) * vdim + j];

    auto fetch = [&](int chunk, float* buf) {
        const int first = chunk * CH, n = min(CH, count - first);
        constexpr int PIECES = PER_TOKEN / 4;                      // 16-byte pieces of a token's data
        for (int e = threadIdx.x; e < CH * PIECES; e += blockDim.x) {
            const int tt = e / PIECES, c = 4 * (e % PIECES);
            float* dst = buf + tt * PER_TOKEN + c;
            if (tt >= n) { *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f); continue; }
            const size_t at = (size_t)(row0 + first + tt) * p.heads + head;
            if (c < DIM) cp_async16(dst, p.kt + at * DIM + c);
            else if (c < 2 * DIM) cp_async16(dst, p.qt + at * DIM + (c - DIM));
            else if (c < 3 * DIM) cp_async16(dst, p.kb + at * DIM + (c - 2 * DIM));
            else if (c < 3 * DIM + AB) cp_async16(dst, p.ab + at * AB + (c - 3 * DIM));
            else cp_async16(dst, p.v + at * vdim + blockIdx.x * FAST_COLS + (c - 3 * DIM - AB));
        }
        for (int e = threadIdx.x; e < DIM / 4; e += blockDim.x)
            cp_async16(buf + CH * PER_TOKEN + 4 * e, p.gc + ((size_t)(row0 + first) * p.heads + head) * DIM + 4 * e);
        cp_async_commit();
    };
    const int chunks = (count + CH - 1) / CH;
    if (chunks > 0) fetch(0, buffers[0]);
    for (int chunk = 0; chunk < chunks; ++chunk) {
        cp_async_wait_all();
        __syncthreads();
        if (chunk + 1 < chunks) fetch(chunk + 1, buffers[(chunk + 1) & 1]);
        const float* buf = buffers[chunk & 1];
        const int n = min(CH, count - chunk * CH);
        // this lane's share of S0^T (e^L k_t) and S0^T (e^L q_t) for every token of the chunk
        float pred[CH], read[CH];
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int q = 0; q < RQ; ++q) {
                const float4 kt = *reinterpret_cast<const float4*>(buf + tt * PER_TOKEN + 4 * (row_lane + LPC * q));
                const float4 qt = *reinterpret_cast<const float4*>(buf + tt * PER_TOKEN + DIM + 4 * (row_lane + LPC * q));
                a += kt.x * s[q][0] + kt.y * s[q][1] + kt.z * s[q][2] + kt.w * s[q][3];
                b += qt.x * s[q][0] + qt.y * s[q][1] + qt.z * s[q][2] + qt.w * s[q][3];
            }
            pred[tt] = a;
            read[tt] = b;
        }
        // sums over the lanes of the column, token l's landing in lane l: halve the tokens a lane carries four times
        if (LPC == 32) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                pred[tt] += __shfl_xor_sync(0xffffffffu, pred[tt], 16);
                read[tt] += __shfl_xor_sync(0xffffffffu, read[tt], 16);
            }
        }
#pragma unroll
        for (int step = 8; step >= 1; step >>= 1) {
            const bool upper = (l & step) != 0;
#pragma unroll
            for (int i = 0; i < step; ++i) {
                const float give_p = upper ? pred[i] : pred[i + step], keep_p = upper ? pred[i + step] : pred[i];
                const float give_r = upper ? read[i] : read[i + step], keep_r = upper ? read[i + step] : read[i];
                pred[i] = keep_p + __shfl_xor_sync(0xffffffffu, give_p, step);
                read[i] = keep_r + __shfl_xor_sync(0xffffffffu, give_r, step);
            }
        }
        // lane l now holds token l's sums in pred[0] and read[0]
        float mine_p = pred[0], mine_r = read[0];
        const float beta = buf[l * PER_TOKEN + 3 * DIM + 2 * CH];
        const float vj = buf[l * PER_TOKEN + 3 * DIM + AB + col];
        float u[CH];
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
            const float candidate = beta * (vj - mine_p);                       // u of this lane's token, final once tt reaches it
            u[tt] = __shfl_sync(0xffffffffu, candidate, LPC == 32 ? tt : (lane & 16) + tt);
            const float* column = buf + tt * PER_TOKEN + 3 * DIM;              // what u_tt adds to the later tokens
            mine_p += column[l] * u[tt];                                        // zero unless l > tt
            mine_r += column[CH + l] * u[tt];                                   // zero unless l >= tt
        }
        if (row_lane < n) p.out[((size_t)(row0 + chunk * CH + l) * p.heads + head) * vdim + j] = mine_r;
        // the state behind the chunk
        const float* gc = buf + CH * PER_TOKEN;
#pragma unroll
        for (int q = 0; q < RQ; ++q) {
            const float4 g = *reinterpret_cast<const float4*>(gc + 4 * (row_lane + LPC * q));
            float acc[4] = {g.x * s[q][0], g.y * s[q][1], g.z * s[q][2], g.w * s[q][3]};
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                const float4 kb = *reinterpret_cast<const float4*>(buf + tt * PER_TOKEN + 2 * DIM + 4 * (row_lane + LPC * q));
                acc[0] += kb.x * u[tt]; acc[1] += kb.y * u[tt]; acc[2] += kb.z * u[tt]; acc[3] += kb.w * u[tt];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) s[q][e] = acc[e];
        }
    }
#pragma unroll
    for (int q = 0; q < RQ; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) state[(size_t)(4 * (row_lane + LPC * q) + e) * vdim + j] = s[q][e];
}

// out[t, h, :] = o / sqrt(mean(o^2) + eps) * w * gate[t, h, :].  One warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                              const float* __restrict__ w, float eps, TO* __restrict__ out,
                                                              long long items, int vdim) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= items) return;
    const float* src = o + item * vdim;
    float sq = 0.f;
    for (int i = lane; i < vdim; i += 32) { const float x = src[i]; sq += x * x; }
    const float inv = rsqrtf(warp_sum(sq) / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32)
        out[item * vdim + i] = from_float<TO>(src[i] * inv * w[i] * (gate ? gate[item * vdim + i] : 1.f));
}

// ----------------------------------------------------------------------------- the recurrence, few tokens per sequence
// A step of one token (or a few) per sequence costs the state's bytes, so the kernel is laid out for them: a block
// owns STEP_COLS = 32 neighbouring columns of one head's state and threadIdx.x = row group * 32 + column, so a warp reads
// and writes 128 consecutive bytes of a row; a thread keeps RPT consecutive rows of its column in registers, and the
// two sums over rows (the prediction, the read-out) meet in shared memory.  grid (column blocks, heads, sequences).
constexpr int STEP_COLS = 32;

template <int RPT>
__global__ void __launch_bounds__(512) delta_step_kernel(const ScanParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int dim = p.dim, vdim = p.vdim;
    const int groups = blockDim.x / STEP_COLS;
    float* ks = sm;                     // [dim]
    float* qs = ks + dim;               // [dim]
    float* gs = qs + dim;               // [dim] decays
    float* sums = gs + dim;             // [groups][STEP_COLS]
    const int head = blockIdx.y, seq = blockIdx.z;
    const int kvh = head / (p.heads / p.kv_heads);
    const int c = threadIdx.x % STEP_COLS, rg = threadIdx.x / STEP_COLS;
    const int j = blockIdx.x * STEP_COLS + c;
    const bool live = j < vdim;
    const int row0 = p.seq_start[seq], count = p.seq_start[seq + 1] - row0;
    float* state = p.state + ((size_t)p.slots[seq] * p.heads + head) * dim * vdim;
    float s[RPT];
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
        const int i = rg * RPT + m;
        s[m] = (live && i < dim) ? state[(size_t)i * vdim + j] : 0.f;
    }
    for (int tt = 0; tt < count; ++tt) {
        const size_t t = (size_t)(row0 + tt);
        __syncthreads();                                              // everyone is done with the token before
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            ks[i] = p.k[(t * p.kv_heads + kvh) * dim + i];
            qs[i] = p.q[(t * p.kv_heads + kvh) * dim + i];
            gs[i] = expf(p.decay[(t * p.heads + head) * dim + i]);
        }
        const float vj = live ? p.v[(t * p.heads + head) * vdim + j] : 0.f;
        const float beta = p.beta[t * p.heads + head];
        __syncthreads();
        float part = 0.f;
#pragma unroll
        for (int m = 0; m < RPT; ++m) {
            const int i = rg * RPT + m;
            if (i < dim) { s[m] *= gs[i]; part += s[m] * ks[i]; }
        }
        sums[rg * STEP_COLS + c] = part;
        __syncthreads();
        float pred = 0.f;
        for (int g = 0; g < groups; ++g) pred += sums[g * STEP_COLS + c];
        const float u = beta * (vj - pred);
        part = 0.f;
#pragma unroll
        for (int m = 0; m < RPT; ++m) {
            const int i = rg * RPT + m;
            if (i < dim) { s[m] += ks[i] * u; part += s[m] * qs[i]; }
        }
        __syncthreads();                                              // the predictions have been read
        sums[rg * STEP_COLS + c] = part;
        __syncthreads();
        if (rg == 0 && live) {
            float o = 0.f;
            for (int g = 0; g < groups; ++g) o += sums[g * STEP_COLS + c];
            p.out[(t * p.heads + head) * vdim + j] = o;
        }
    }
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
        const int i = rg * RPT + m;
        if (live && i < dim) state[(size_t)i * vdim + j] = s[m];
    }
}

template <int RPT>
static int launch_step(const ScanParams& p, int n_seqs, cudaStream_t s) {
    const int groups = (p.dim + RPT - 1) / RPT;
    const size_t smem = ((size_t)3 * p.dim + (size_t)groups * STEP_COLS) * sizeof(float);
    launch_kernel(delta_step_kernel<RPT>, dim3((p.vdim + STEP_COLS - 1) / STEP_COLS, p.heads, n_seqs), dim3(groups * STEP_COLS), smem, s, p);
    QT_CHECK_LAUNCH("delta_step");
    return QT_OK;
}

// ----------------------------------------------------------------------------- entry points
extern "C" int qt_delta_prepare(const float* proj, int n_splits, long long split_stride, int proj_cols, const float* taps,
                                float* kept, const int* token_seq, const int* token_pos, const int* seq_start,
                                const int* seq_past, const int* slots, float* q, float* k, float* v, float* beta, int n_tokens,
                                int n_seqs, int heads, int kv_heads, int dim, int vdim, int n_taps, float unit_eps, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0,
               "delta_prepare: bad sizes T=%d heads=%d kv_heads=%d dim=%d vdim=%d", n_tokens, heads, kv_heads, dim, vdim);
    QT_REQUIRE(n_taps >= 1 && n_taps <= MAX_TAPS, "delta_prepare: a convolution of %d taps (1..%d)", n_taps, MAX_TAPS);
    const int channels = 2 * kv_heads * dim + heads * vdim;
    QT_REQUIRE(proj_cols >= channels + heads && n_splits >= 1, "delta_prepare: a projection of %d columns does not hold q, k, v and beta", proj_cols);
    if (n_tokens == 0) return QT_OK;
    PrepareParams p{proj, n_splits, (size_t)split_stride, proj_cols, taps, kept, token_seq, token_pos, seq_start, seq_past, slots,
                    q, k, v, beta, n_tokens, heads, kv_heads, dim, vdim, n_taps, unit_eps};
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)n_tokens * (2 * kv_heads + heads + 1);
    launch_kernel(delta_prepare_kernel, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, s, p);
    QT_CHECK_LAUNCH("delta_prepare");
    if (n_taps > 1) {
        launch_kernel(conv_keep_kernel, dim3((channels + 127) / 128, n_seqs), dim3(128), 0, s, proj, n_splits, (size_t)split_stride, proj_cols,
                      kept, seq_start, slots, n_seqs, channels, n_taps);
        QT_CHECK_LAUNCH("conv_keep");
    }
    return QT_OK;
}

extern "C" int qt_lowrank(const float* proj, int n_splits, long long split_stride, int proj_cols, int x_offset, int rank,
                          const float* w, const float* bias, const float* rate_log, int per_rate, float* out, int n_tokens,
                          int n_out, int mode, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && n_out > 0 && rank > 0 && x_offset >= 0 && x_offset + rank <= proj_cols && n_splits >= 1,
               "lowrank: bad sizes T=%d N=%d rank=%d at column %d of %d", n_tokens, n_out, rank, x_offset, proj_cols);
    QT_REQUIRE(mode == LR_SIGMOID || (mode == LR_DECAY && rate_log && per_rate > 0), "lowrank: mode %d", mode);
    QT_REQUIRE((size_t)LR_TOKENS * rank * sizeof(float) <= 48 * 1024, "lowrank: %d columns are too many for a tile in shared memory", rank);
    if (n_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (n_tokens <= 16 * LR_TOKENS) {
        const size_t few_smem = ((size_t)LR_TOKENS * rank + 4 * LR_TOKENS * 64) * sizeof(float);
        if (few_smem <= 48 * 1024) {
            const dim3 few_grid((n_out + 63) / 64, (n_tokens + LR_TOKENS - 1) / LR_TOKENS);
            if (mode == LR_DECAY)
                launch_kernel(lowrank_few_kernel<LR_DECAY>, few_grid, dim3(256), few_smem, s, proj, n_splits, (size_t)split_stride, proj_cols, x_offset,
                              rank, w, bias, rate_log, per_rate, out, n_tokens, n_out);
            else
                launch_kernel(lowrank_few_kernel<LR_SIGMOID>, few_grid, dim3(256), few_smem, s, proj, n_splits, (size_t)split_stride, proj_cols, x_offset,
                              rank, w, bias, rate_log, per_rate, out, n_tokens, n_out);
            QT_CHECK_LAUNCH("lowrank");
            return QT_OK;
        }
    }
    const int threads = 256;
    const dim3 grid((n_out + threads - 1) / threads, (n_tokens + LR_TOKENS - 1) / LR_TOKENS);
    const size_t smem = (size_t)LR_TOKENS * rank * sizeof(float);
    if (mode == LR_DECAY)
        launch_kernel(lowrank_kernel<LR_DECAY>, grid, dim3(threads), smem, s, proj, n_splits, (size_t)split_stride, proj_cols, x_offset, rank, w, bias,
                      rate_log, per_rate, out, n_tokens, n_out);
    else
        launch_kernel(lowrank_kernel<LR_SIGMOID>, grid, dim3(threads), smem, s, proj, n_splits, (size_t)split_stride, proj_cols, x_offset, rank, w, bias,
                      rate_log, per_rate, out, n_tokens, n_out);
    QT_CHECK_LAUNCH("lowrank");
    return QT_OK;
}

template <int R>
static int launch_scan(const ScanParams& p, int n_seqs, cudaStream_t s) {
    const size_t smem = 2 * (size_t)SCAN_CHUNK * (3 * p.dim + SCAN_COLS + 1) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(delta_scan_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "delta_scan: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    launch_kernel(delta_scan_kernel<R>, dim3((p.vdim + SCAN_COLS - 1) / SCAN_COLS, p.heads, n_seqs), dim3(SCAN_COLS * SCAN_LANES), smem, s, p);
    QT_CHECK_LAUNCH("delta_scan");
    return QT_OK;
}

extern "C" int qt_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* decay, float* state,
                             float* out, const int* seq_start, const int* slots, int n_seqs, int heads, int kv_heads, int dim,
                             int vdim, void* stream) {
    QT_REQUIRE(n_seqs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && vdim > 0, "delta_scan: bad sizes");
    QT_REQUIRE(dim > 0 && dim <= 512, "delta_scan: %d key channels per head (1..512)", dim);
    QT_REQUIRE(n_seqs <= 65535 && heads <= 65535, "delta_scan: too many sequences or heads for one launch");
    if (n_seqs == 0) return QT_OK;
    ScanParams p{q, k, v, beta, decay, state, out, seq_start, slots, heads, kv_heads, dim, vdim};
    cudaStream_t s = (cudaStream_t)stream;
    static const bool lanes_form = [] { const char* env = getenv("QT_B200_DELTA_STEP"); return env && env[0] == '0'; }();
    if (!lanes_form) {                                                // rows of a column over row groups, 128 bytes of a row per warp
        if (dim <= 64) return launch_step<8>(p, n_seqs, s);
        if (dim <= 256) return launch_step<16>(p, n_seqs, s);
        return launch_step<32>(p, n_seqs, s);
    }
    if (dim <= 32) return launch_scan<4>(p, n_seqs, s);
    if (dim <= 64) return launch_scan<8>(p, n_seqs, s);
    if (dim <= 128) return launch_scan<16>(p, n_seqs, s);
    if (dim <= 256) return launch_scan<32>(p, n_seqs, s);
    return launch_scan<64>(p, n_seqs, s);
}

template <int R>
static int launch_chunk_scan(const ChunkScanParams& p, int n_seqs, cudaStream_t s) {
    const size_t smem = 2 * ((size_t)CH * (3 * p.dim + 2 * CH + SCAN_COLS + 1) + p.dim) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(delta_chunk_scan_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "delta_chunk_scan: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    QT_REQUIRE(smem <= 220 * 1024, "delta_chunk_scan: %d key channels per head need more shared memory than a block has", p.dim);
    launch_kernel(delta_chunk_scan_kernel<R>, dim3((p.vdim + SCAN_COLS - 1) / SCAN_COLS, p.heads, n_seqs), dim3(SCAN_COLS * SCAN_LANES), smem, s, p);
    QT_CHECK_LAUNCH("delta_chunk_scan");
    return QT_OK;
}

template <int LPC, int RQ>
static int launch_chunk_scan_fast(const ChunkScanParams& p, int n_seqs, cudaStream_t s) {
    const size_t smem = 2 * ((size_t)CH * (3 * 4 * LPC * RQ + AB + FAST_COLS) + 4 * LPC * RQ) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(delta_chunk_scan_fast_kernel<LPC, RQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "delta_chunk_scan: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    launch_kernel(delta_chunk_scan_fast_kernel<LPC, RQ>, dim3(p.vdim / FAST_COLS, p.heads, n_seqs), dim3(FAST_COLS * LPC), smem, s, p);
    QT_CHECK_LAUNCH("delta_chunk_scan");
    return QT_OK;
}

// The recurrence in chunks (steps of many tokens per sequence).  Scratch of the caller: kt, qt, kb, gc [T, heads, dim] and
// ab [T, heads, 36], float.  `max_tokens` is the most tokens any sequence of the step has.
extern "C" int qt_delta_scan_chunked(const float* q, const float* k, const float* v, const float* beta, const float* log_decay,
                                     float* state, float* out, float* kt, float* qt, float* kb, float* gc, float* ab,
                                     const int* seq_start, const int* slots, int n_seqs, int max_tokens, int heads, int kv_heads,
                                     int dim, int vdim, void* stream) {
    QT_REQUIRE(n_seqs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && vdim > 0 && max_tokens >= 0, "delta_scan_chunked: bad sizes");
    QT_REQUIRE(dim > 0 && dim <= 256, "delta_scan_chunked: %d key channels per head (1..256)", dim);
    QT_REQUIRE(n_seqs <= 65535 && heads <= 65535, "delta_scan_chunked: too many sequences or heads for one launch");
    if (n_seqs == 0 || max_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    ChunkParams cp{q, k, log_decay, kt, qt, kb, gc, beta, ab, seq_start, heads, kv_heads, dim};
    const size_t smem = 3 * (size_t)CH * dim * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(delta_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "delta_chunk_prepare: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    launch_kernel(delta_chunk_prepare_kernel, dim3((max_tokens + CH - 1) / CH, heads, n_seqs), dim3(128), smem, s, cp);
    QT_CHECK_LAUNCH("delta_chunk_prepare");
    ChunkScanParams sp{kt, qt, kb, gc, ab, v, beta, state, out, seq_start, slots, heads, dim, vdim};
    static const bool plain_only = [] { const char* env = getenv("QT_B200_DELTA_FAST"); return env && env[0] == '0'; }();
    const bool aligned = ((uintptr_t)kt % 16 == 0) && ((uintptr_t)qt % 16 == 0) && ((uintptr_t)kb % 16 == 0) && ((uintptr_t)gc % 16 == 0) &&
                         ((uintptr_t)ab % 16 == 0) && ((uintptr_t)v % 16 == 0);
    if (!plain_only && aligned && dim % 64 == 0 && dim <= 256 && vdim % FAST_COLS == 0) {
        // 16 lanes per column unless QT_B200_DELTA_LANES=32: a warp per column measured 3 to 7 % slower in a prefill of 2,048 tokens
        static const bool half_warps = [] { const char* env = getenv("QT_B200_DELTA_LANES"); return !(env && env[0] == '3' && env[1] == '2'); }();
        if (dim == 64) return launch_chunk_scan_fast<16, 1>(sp, n_seqs, s);
        if (dim == 128) return half_warps ? launch_chunk_scan_fast<16, 2>(sp, n_seqs, s) : launch_chunk_scan_fast<32, 1>(sp, n_seqs, s);
        if (dim == 192) return launch_chunk_scan_fast<16, 3>(sp, n_seqs, s);
        return half_warps ? launch_chunk_scan_fast<16, 4>(sp, n_seqs, s) : launch_chunk_scan_fast<32, 2>(sp, n_seqs, s);
    }
    if (dim <= 32) return launch_chunk_scan<4>(sp, n_seqs, s);
    if (dim <= 64) return launch_chunk_scan<8>(sp, n_seqs, s);
    if (dim <= 128) return launch_chunk_scan<16>(sp, n_seqs, s);
    return launch_chunk_scan<32>(sp, n_seqs, s);
}

extern "C" int qt_gated_head_norm(const float* o, const float* gate, const float* w, float eps, void* out, int out_dtype,
                                  int n_tokens, int heads, int vdim, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && heads > 0 && vdim > 0, "gated_head_norm: bad sizes");
    if (n_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)n_tokens * heads;
    return QT_DISPATCH_DTYPE(out_dtype, "gated_head_norm", {
        launch_kernel(gated_head_norm_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, s, o, gate, w, eps, (T*)out, items, vdim);
        QT_CHECK_LAUNCH("gated_head_norm");
        return QT_OK;
    });
}

QT_DEFINE_LAST_ERROR(delta_rule)
