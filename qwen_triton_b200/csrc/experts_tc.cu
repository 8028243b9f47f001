// The two products of table-chosen experts for many tokens, on the fifth-generation tensor cores.
//
// The rows (token, expert pairs) arrive ordered by expert, every expert's run padded to whole tiles of 128 rows
// (experts.cu), so a tile's rows all take one expert's weight: Y[rows of the tile, :] = X[rows, :] * W[e]^T with e read
// from `tile_expert`.  A tile beyond the last run (-1) leaves at once.  The weights of all experts are one matrix
// [E * N, K]; a weight tile of 128 rows that reaches past its expert's N rows reads the next expert's (or zeros past
// the end), and the epilogue drops those columns.
//
// The rows are the MMA's M (128 per block), the weight rows its N (256 where there is such a tile for every SM, else 128): a thread
// of the epilogue holds 32 consecutive output features of one row per tcgen05.ld, applies the activation where asked
// and stores 16 bytes at a time.  Two blocks share an SM (96 KB of shared memory and at most 256 columns of tensor
// memory each) at N = 128 with a three-stage ring, so one's epilogue runs under the other's MMAs; at N = 256 a block has
// the SM to itself, a four-stage ring and two accumulators, and walks several tiles (expert_gemm_persistent_kernel).
// TMA (128-byte swizzle) stages 64-element K slices in a ring; one elected thread issues tcgen05.mma, the
// accumulator lives in tensor memory.  Warp roles and the bounded waits are those of gemm_tc.cu.
#include "tc_common.cuh"

using namespace qt;
using namespace qt_tc;

namespace {

constexpr int BM = 128;        // rows per tile = MMA M
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr uint32_t A_BYTES = BM * BK * 2;

__device__ __forceinline__ void store8(float* dst, const float (&f)[8]) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* dst, const float (&f)[8]) {
    uint4 packed;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(f[0], f[1]); packed.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[2], f[3]); packed.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[4], f[5]); packed.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(f[6], f[7]); packed.w = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint4*>(dst) = packed;
}

template <typename TO, bool ACT, int BN, int STAGES>
__global__ void __launch_bounds__(THREADS) expert_gemm_kernel(const __grid_constant__ CUtensorMap map_x,
                                                              const __grid_constant__ CUtensorMap map_w, TO* __restrict__ out,
                                                              const int* __restrict__ tile_expert, int n_out, int kb_total,
                                                              int w_tiles, int act, int* status) {
    constexpr uint32_t B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    // instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N = BN, M = 128
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    pdl_launch_dependents();
    pdl_wait();                                                    // the routing and the rows come from the kernels before
    const int x_tile = blockIdx.x / w_tiles, w_tile = blockIdx.x % w_tiles;
    const int expert = tile_expert[x_tile];
    if (expert < 0) return;                                        // the whole block: nothing is set up yet

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                  // swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (base - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE_BYTES);
    const uint32_t full0 = base + STAGES * STAGE_BYTES, empty0 = full0 + 8 * STAGES, tmem_full = empty0 + 8 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int x0 = x_tile * BM, w0 = expert * n_out + w_tile * BN;

    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_w);
        prefetch_tensor_map(&map_x);
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < kb_total; ++i) {
                if (i >= STAGES && !mbar_wait(empty0 + 8 * s, phase ^ 1u, status, 1)) break;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                const uint32_t dst = base + s * STAGE_BYTES;
                tma_load_2d(dst, &map_x, full0 + 8 * s, i * BK, x0);
                tma_load_2d(dst + A_BYTES, &map_w, full0 + 8 * s, i * BK, w0);
                if (++s == STAGES) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint64_t a_desc0 = operand_desc(base), b_desc0 = operand_desc(base + A_BYTES);
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < kb_total; ++i) {
                if (!mbar_wait(full0 + 8 * s, phase, status, 2)) break;
                tc_fence_after();
                const uint64_t a_desc = a_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
                const uint64_t b_desc = b_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)      // 32 bytes further along K inside the swizzled row
                    umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);
                if (++s == STAGES) { s = 0; phase ^= 1u; }
            }
            umma_commit(tmem_full);
        }
    } else {
        const int quarter = warp & 3;                      // the accumulator lanes this warp may read
        const bool ready = mbar_wait(tmem_full, 0, status, 3);
        tc_fence_after();
        TO* dst = out + (size_t)(x0 + quarter * 32 + lane) * n_out;
        if (ready) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                const int f0 = w_tile * BN + c;
                if (f0 >= n_out) break;                    // the same for the whole warp
                uint32_t v[32];
                tmem_load32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (f0 + 8 * g >= n_out) break;        // n_out is a multiple of 8
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float a = __uint_as_float(v[8 * g + j]);
                        f[j] = ACT ? gate_activation<false>(a, act) : a;
                    }
                    store8(dst + f0 + 8 * g, f);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*(volatile int*)status != 0) {                     // a wait gave up: let copies in flight land before the block leaves
        const unsigned long long t0 = global_timer();
        while (global_timer() - t0 < 2000000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// The same product for many tiles: one block per SM walks the tiles block, block + blocks, ... with 128 x 256 tiles, a
// four-stage ring that runs on across tiles and two accumulators in tensor memory (all 512 columns), so that the
// epilogue of a tile runs under the MMAs of the next and the ring never drains between tiles.  Tiles of the padding
// beyond the last run (-1) are skipped by every role alike.
constexpr int PBN = 256, PSTAGES = 4;
constexpr uint32_t P_B_BYTES = PBN * BK * 2, P_STAGE_BYTES = A_BYTES + P_B_BYTES;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <typename TO, bool ACT>
__global__ void __launch_bounds__(THREADS, 1) expert_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                            const __grid_constant__ CUtensorMap map_w, TO* __restrict__ out,
                                                                            const int* __restrict__ tile_expert, int n_out, int kb_total,
                                                                            int w_tiles, int total_items, int act, int* status) {
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PBN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    pdl_launch_dependents();
    pdl_wait();                                                    // the routing and the rows come from the kernels before
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)PSTAGES * P_STAGE_BYTES);
    const uint32_t full0 = base + PSTAGES * P_STAGE_BYTES, empty0 = full0 + 8 * PSTAGES;
    const uint32_t acc_full0 = empty0 + 8 * PSTAGES, acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PSTAGES + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_w);
        prefetch_tensor_map(&map_x);
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                const int x_tile = item / w_tiles, w_tile = item % w_tiles;
                const int expert = tile_expert[x_tile];
                if (expert < 0) continue;
                const int x0 = x_tile * BM, w0 = expert * n_out + w_tile * PBN;
                for (int i = 0; i < kb_total; ++i) {
                    // a stage that was never filled counts as free: the wait on the phase before a barrier's first passes at once
                    if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, status, 1)) { ok = false; break; }
                    mbar_expect_tx(full0 + 8 * s, P_STAGE_BYTES);
                    const uint32_t dst = base + s * P_STAGE_BYTES;
                    tma_load_2d(dst, &map_x, full0 + 8 * s, i * BK, x0);
                    tma_load_2d(dst + A_BYTES, &map_w, full0 + 8 * s, i * BK, w0);
                    if (++s == PSTAGES) { s = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint64_t a_desc0 = operand_desc(base), b_desc0 = operand_desc(base + A_BYTES);
            int s = 0, t = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                if (tile_expert[item / w_tiles] < 0) continue;
                const int a = t & 1;
                // the accumulator is free once the epilogue of the tile two before this one has read it
                if (!mbar_wait(acc_empty0 + 8 * a, ((uint32_t)(t >> 1) & 1u) ^ 1u, status, 4)) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(a * PBN);
                for (int i = 0; i < kb_total; ++i) {
                    if (!mbar_wait(full0 + 8 * s, phase, status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t a_desc = a_desc0 + (uint64_t)(s * (P_STAGE_BYTES >> 4));
                    const uint64_t b_desc = b_desc0 + (uint64_t)(s * (P_STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(acc, a_desc + 2 * k, b_desc + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);
                    if (++s == PSTAGES) { s = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(acc_full0 + 8 * a);
                ++t;
            }
        }
    } else {
        const int quarter = warp & 3;
        int t = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
            const int x_tile = item / w_tiles, w_tile = item % w_tiles;
            if (tile_expert[x_tile] < 0) continue;
            const int a = t & 1;
            if (!mbar_wait(acc_full0 + 8 * a, (uint32_t)(t >> 1) & 1u, status, 3)) break;
            tc_fence_after();
            TO* dst = out + (size_t)(x_tile * BM + quarter * 32 + lane) * n_out;
#pragma unroll 1
            for (int c = 0; c < PBN; c += 32) {
                const int f0 = w_tile * PBN + c;
                if (f0 >= n_out) break;
                uint32_t v[32];
                tmem_load32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * PBN + c), v);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (f0 + 8 * g >= n_out) break;
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float x = __uint_as_float(v[8 * g + j]);
                        f[j] = ACT ? gate_activation<false>(x, act) : x;
                    }
                    store8(dst + f0 + 8 * g, f);
                }
            }
            tc_fence_before();                              // the reads of this accumulator are done: hand it back
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * a);
            ++t;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*(volatile int*)status != 0) {
        const unsigned long long t0 = global_timer();
        while (global_timer() - t0 < 2000000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <typename TO, bool ACT>
int launch_persistent(const void* x, const void* w, TO* out, const int* tile_expert, int max_tiles, int experts, int n_out, int K, int act,
                      int* status, cudaStream_t stream) {
    CUtensorMap map_x, map_w;
    int rc = tensor_map(&map_x, x, (uint64_t)max_tiles * BM, (uint64_t)K, BM);
    if (rc) return rc;
    rc = tensor_map(&map_w, w, (uint64_t)experts * n_out, (uint64_t)K, PBN);
    if (rc) return rc;
    const size_t smem = (size_t)PSTAGES * P_STAGE_BYTES + 1024 + (2 * PSTAGES + 4) * 8 + 16;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(expert_gemm_persistent_kernel<TO, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "expert_gemm: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int w_tiles = (n_out + PBN - 1) / PBN, kb_total = (K + BK - 1) / BK;
    const long long items = (long long)max_tiles * w_tiles;
    QT_REQUIRE(items < (1ll << 31), "expert_gemm: too many tiles for one launch");
    const int blocks = (int)(items < sm_count() ? items : sm_count());
    launch_kernel(expert_gemm_persistent_kernel<TO, ACT>, dim3((unsigned)blocks), dim3(THREADS), smem, stream, map_x, map_w, out, tile_expert,
                  n_out, kb_total, w_tiles, (int)items, act, status);
    QT_CHECK_LAUNCH("expert_gemm");
    return QT_OK;
}

template <typename TO, bool ACT, int BN, int STAGES>
int launch_tile(const void* x, const void* w, TO* out, const int* tile_expert, int max_tiles, int experts, int n_out, int K, int act, int* status,
                cudaStream_t stream) {
    CUtensorMap map_x, map_w;
    int rc = tensor_map(&map_x, x, (uint64_t)max_tiles * BM, (uint64_t)K, BM);
    if (rc) return rc;
    rc = tensor_map(&map_w, w, (uint64_t)experts * n_out, (uint64_t)K, BN);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + 1024 + (2 * STAGES + 1) * 8 + 16;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(expert_gemm_kernel<TO, ACT, BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "expert_gemm: cannot raise shared memory: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int w_tiles = (n_out + BN - 1) / BN, kb_total = (K + BK - 1) / BK;
    QT_REQUIRE((long long)max_tiles * w_tiles < (1ll << 31), "expert_gemm: too many tiles for one launch");
    launch_kernel(expert_gemm_kernel<TO, ACT, BN, STAGES>, dim3((unsigned)(max_tiles * w_tiles)), dim3(THREADS), smem, stream, map_x, map_w, out,
                  tile_expert, n_out, kb_total, w_tiles, act, status);
    QT_CHECK_LAUNCH("expert_gemm");
    return QT_OK;
}

template <typename TO, bool ACT>
int launch(const void* x, const void* w, TO* out, const int* tile_expert, int max_tiles, int experts, int n_out, int K, int act, int* status,
           cudaStream_t stream) {
    // 128 x 256 tiles fetch a third less per flop than 128 x 128 ones.  Where there is a tile of them for every SM the
    // persistent kernel takes the product: 16 experts of 4,096 x 2,048, 2 per token: 1,170 and 1,250 TFLOP/s for up and
    // down at 8,192 tokens (907 and 1,065 with a launch per tile and one accumulator), 621 and 714 at 2,048 tokens
    // (555 and 652; 128 x 128 tiles, two blocks to an SM: 600 and 660).  Fewer tiles than SMs: the small tiles.
    // QT_B200_EXPERTS_PERSISTENT=0 and QT_B200_EXPERTS_WIDE_WAVES (tiles per SM from which the wide form runs) are the switches.
    const long long wide_items = (long long)max_tiles * ((n_out + 255) / 256);
    static const bool persistent = [] { const char* env = getenv("QT_B200_EXPERTS_PERSISTENT"); return !(env && env[0] == '0'); }();
    static const int waves = [] { const char* env = getenv("QT_B200_EXPERTS_WIDE_WAVES"); return env ? atoi(env) : 1; }();
    if (n_out > 128 && wide_items >= (long long)waves * sm_count()) {
        if (persistent) return launch_persistent<TO, ACT>(x, w, out, tile_expert, max_tiles, experts, n_out, K, act, status, stream);
        return launch_tile<TO, ACT, 256, 4>(x, w, out, tile_expert, max_tiles, experts, n_out, K, act, status, stream);
    }
    return launch_tile<TO, ACT, 128, 3>(x, w, out, tile_expert, max_tiles, experts, n_out, K, act, status, stream);
}

}  // namespace

// out [max_tiles * 128, n_out] = act?(x [max_tiles * 128, K] * w[tile's expert] [n_out, K]^T), w being [experts * n_out, K].
// `act` < 0: no activation.  Codes in `status`: as in gemm_tc.cu (1 = the TMA producer, 2 = the MMA issuer, 3 = the epilogue).
extern "C" int qt_expert_gemm(const void* x, const void* w, void* out, int out_dtype, const int* tile_expert, int max_tiles, int experts,
                              int n_out, int K, int act, int* status, void* stream) {
    QT_REQUIRE(max_tiles > 0 && experts > 0 && n_out > 0 && K > 0, "expert_gemm: bad sizes tiles=%d E=%d N=%d K=%d", max_tiles, experts, n_out, K);
    QT_REQUIRE(K % 8 == 0 && n_out % 8 == 0, "expert_gemm: K=%d and N=%d must be multiples of 8 (16-byte rows for TMA and for the stores)", K, n_out);
    QT_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0), "expert_gemm: operands must be 16-byte aligned");
    QT_REQUIRE(act < QT_ACT_COUNT, "expert_gemm: unknown activation code %d", act);
    QT_REQUIRE(status != nullptr && tile_expert != nullptr, "expert_gemm: a status word and the tiles' experts are required");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == QT_BF16 && act >= 0) return launch<__nv_bfloat16, true>(x, w, (__nv_bfloat16*)out, tile_expert, max_tiles, experts, n_out, K, act, status, s);
    if (out_dtype == QT_BF16) return launch<__nv_bfloat16, false>(x, w, (__nv_bfloat16*)out, tile_expert, max_tiles, experts, n_out, K, 0, status, s);
    if (out_dtype == QT_F32 && act < 0) return launch<float, false>(x, w, (float*)out, tile_expert, max_tiles, experts, n_out, K, 0, status, s);
    QT_FAIL(QT_ERR_ARG, "expert_gemm: output type %d%s is not offered", out_dtype, act >= 0 ? " with an activation" : "");
}

QT_DEFINE_LAST_ERROR(experts_tc)
