// Feed-forward experts chosen per token by a table: each token runs the `top` experts that the table's row of its
// token id names, out[t] = sum_k weight_k * W_down[e_k] act(W_up[e_k] x[t]).  The routing is read on the device
// (token ids and table are device arrays), so a step with these kernels has the same launches whatever the tokens
// are and can be captured in a CUDA graph.
//
// Two forms.  Few tokens (a decode step): one pass of matrix-vector products per (token, expert) pair, the expert's
// rows streamed once per pair.  Many tokens: the pairs are ordered by expert on the device (count, offsets, scatter;
// every expert's run padded to whole tiles of rows), and the two products run tile by tile, a tile's rows all of one
// expert, so that an expert's weights are read once per tile instead of once per pair.
#include "common.cuh"

#include <math.h>

using namespace qt;

// ----------------------------------------------------------------------------- few tokens: per pair
constexpr int EV_WARPS = 8;
constexpr int EV_FEATS = 4;        // output features per warp and pass

struct ExpertParams {
    const void* x;            // [T, width] normed rows
    const int* token_ids;     // [T]
    const int* table;         // [vocab, top]
    const void* up;           // [E, ff, width]
    const void* down;         // [E, width, ff]
    void* mid;                // [T * top, ff] activations
    float* out;               // [T, width] float
    int n_tokens, vocab, top, experts, width, ff, act;
    float pair_weight;        // weight of every chosen expert (1 / top for an unweighted mean)
};

__device__ __forceinline__ int expert_of(const ExpertParams& p, int t, int k) {
    int id = p.token_ids[t];
    id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
    int e = p.table[(size_t)id * p.top + k];
    return e < 0 ? 0 : (e >= p.experts ? p.experts - 1 : e);          // never read outside the weights
}

// mid[pair, f] = act(W_up[e][f, :] . x[t, :]).  grid (pairs, feature blocks); x[t] in shared memory as float.
template <typename T>
__global__ void __launch_bounds__(EV_WARPS * 32) expert_up_kernel(const ExpertParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];
    const int pair = blockIdx.x, t = pair / p.top, k = pair % p.top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* x = (const T*)p.x + (size_t)t * p.width;
    for (int i = threadIdx.x; i < p.width; i += blockDim.x) xs[i] = to_float(x[i]);
    __syncthreads();
    const int e = expert_of(p, t, k);
    const T* w = (const T*)p.up + (size_t)e * p.ff * p.width;
    T* mid = (T*)p.mid + (size_t)pair * p.ff;
    const int f0 = (blockIdx.y * EV_WARPS + warp) * EV_FEATS;
    float acc[EV_FEATS];
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j) acc[j] = 0.f;
    for (int i = lane; i < p.width; i += 32) {
        const float xv = xs[i];
#pragma unroll
        for (int j = 0; j < EV_FEATS; ++j)
            if (f0 + j < p.ff) acc[j] += to_float(w[(size_t)(f0 + j) * p.width + i]) * xv;
    }
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j) {
        const float total = warp_sum(acc[j]);
        if (lane == 0 && f0 + j < p.ff) mid[f0 + j] = from_float<T>(gate_activation<false>(total, p.act));
    }
}

// out[t, c] = pair_weight * sum_k W_down[e_k][c, :] . mid[t * top + k, :].  grid (tokens, column blocks).
template <typename T>
__global__ void __launch_bounds__(EV_WARPS * 32) expert_down_kernel(const ExpertParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float ms[];                 // [top, ff]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* mid = (const T*)p.mid + (size_t)t * p.top * p.ff;
    for (int i = threadIdx.x; i < p.top * p.ff; i += blockDim.x) ms[i] = to_float(mid[i]);
    __syncthreads();
    const int c0 = (blockIdx.y * EV_WARPS + warp) * EV_FEATS;
    float acc[EV_FEATS];
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j) acc[j] = 0.f;
    for (int k = 0; k < p.top; ++k) {
        const int e = expert_of(p, t, k);
        const T* w = (const T*)p.down + (size_t)e * p.width * p.ff;
        const float* m = ms + k * p.ff;
        for (int i = lane; i < p.ff; i += 32) {
            const float mv = m[i];
#pragma unroll
            for (int j = 0; j < EV_FEATS; ++j)
                if (c0 + j < p.width) acc[j] += to_float(w[(size_t)(c0 + j) * p.ff + i]) * mv;
        }
    }
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j) {
        const float total = warp_sum(acc[j]);
        if (lane == 0 && c0 + j < p.width) p.out[(size_t)t * p.width + c0 + j] = total * p.pair_weight;
    }
}

static int check_experts(const char* name, int n_tokens, int vocab, int top, int experts, int width, int ff, int act) {
    QT_REQUIRE(n_tokens >= 0 && vocab > 0 && top > 0 && experts > 0 && top <= experts, "%s: bad routing sizes T=%d V=%d top=%d E=%d", name, n_tokens, vocab, top, experts);
    QT_REQUIRE(width > 0 && ff > 0, "%s: bad sizes width=%d ff=%d", name, width, ff);
    QT_REQUIRE(act >= 0 && act < QT_ACT_COUNT, "%s: unknown activation code %d", name, act);
    return QT_OK;
}

extern "C" int qt_experts_by_pair(const void* x, const int* token_ids, const int* table, const void* up, const void* down, void* mid,
                                  float* out, int dtype, int n_tokens, int vocab, int top, int experts, int width, int ff, int act,
                                  float pair_weight, void* stream) {
    int rc = check_experts("experts_by_pair", n_tokens, vocab, top, experts, width, ff, act);
    if (rc) return rc;
    if (n_tokens == 0) return QT_OK;
    QT_REQUIRE((size_t)width * 4 <= 200 * 1024 && (size_t)top * ff * 4 <= 200 * 1024, "experts_by_pair: a row of %d or %d x %d floats does not fit shared memory", width, top, ff);
    ExpertParams p{x, token_ids, table, up, down, mid, out, n_tokens, vocab, top, experts, width, ff, act, pair_weight};
    cudaStream_t s = (cudaStream_t)stream;
    const int per_block = EV_WARPS * EV_FEATS;
    return QT_DISPATCH_DTYPE(dtype, "experts_by_pair", {
        const size_t smem_up = (size_t)width * sizeof(float), smem_down = (size_t)top * ff * sizeof(float);
        if (smem_up > 48 * 1024) cudaFuncSetAttribute(expert_up_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
        if (smem_down > 48 * 1024) cudaFuncSetAttribute(expert_down_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
        launch_kernel(expert_up_kernel<T>, dim3(n_tokens * top, (ff + per_block - 1) / per_block), dim3(EV_WARPS * 32), smem_up, s, p);
        QT_CHECK_LAUNCH("expert_up");
        launch_kernel(expert_down_kernel<T>, dim3(n_tokens, (width + per_block - 1) / per_block), dim3(EV_WARPS * 32), smem_down, s, p);
        QT_CHECK_LAUNCH("expert_down");
        return QT_OK;
    });
}

QT_DEFINE_LAST_ERROR(experts)
