// The experts' grouped products in bfloat16 on the tensor cores (tcgen05 + TMA), over the
// plan that moe.cu makes: a tile of sorted (token, choice) rows belongs to one expert.
//
// One CTA per (128 weight rows of the tile's expert, one tile of 64 or 128 sorted rows: the
// plan's tile; 128 where experts have rows enough, since a product of N 128 feeds the
// tensor pipe with half the bytes per flop of one of N 64).  The weight rows
// are the M side (the experts' matrices are stacked [E * N, K], so an expert is a row
// offset in one tensor map), the tile's rows the N side; both come by TMA with the 128-byte
// swizzle into a ring of stages, the products accumulate in tensor memory, and four
// warps read the accumulator back, one output feature per thread, and pass the tile
// through shared memory so that rows leave in 16-byte pieces:
//   gated:  z[pos, f] = act(gate) * up, two accumulators side by side, bfloat16 out;
//   plain:  out[dst[pos], f] = w[pos] * acc, 32-bit out (the down product, scattered to
//           [choice, token] and scaled by the pair's weight).
// Rows of padding (tok[pos] < 0) are computed and dropped.  The left operand's rows must
// lie in sorted order ([rows, K] dense enough for TMA: K and the row stride multiples of
// 8); agv_moe_gather_rows brings a step's tokens into that order.
//
// Which expert a tile belongs to is decided on the device by the plan, so nothing is
// requested before the wait for the kernels before; every wait on a barrier is bounded
// and leaves a code for agv_moe_tc_status.
#include "tcgen05.cuh"
#include <type_traits>

namespace {
using namespace tc5;

constexpr int MT_M = 128;          // weight rows per CTA
constexpr int MT_K = 64;           // 64 bf16 = one 128-byte swizzle row
constexpr int MT_THREADS = 192;

__device__ int g_moe_status = 0;   // 0 ok; else (role << 8) | stage of the first wait that gave up

template <bool GATED, int MT_N>
struct MTile {
    // The plain form (the down product: a short K, a large 32-bit tile to write) keeps its
    // ring small enough for two CTAs to share an SM, so that one's epilogue runs under the
    // other's products; the gated form has a long K and takes the SM alone.
    static constexpr int STAGES = GATED ? (MT_N == 128 ? 2 : 4) : 3;
    static constexpr int A_BYTES = MT_M * MT_K * 2;
    static constexpr int B_BYTES = MT_N * MT_K * 2;
    static constexpr int STAGE_BYTES = A_BYTES * (GATED ? 2 : 1) + B_BYTES;
    static constexpr int TMEM_COLS = GATED ? 2 * MT_N : MT_N;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 2048 /*barriers, rows*/;
};

__device__ __forceinline__ float mt_act(float t, int act) {
    if (act == 1) return __fdividef(t, 1.0f + __expf(-t));
    const float u = 0.7978845608028654f * (t + 0.044715f * t * t * t);
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(u));
    return 0.5f * t * (1.0f + th);
}

template <bool GATED, int MT_N>
__global__ void __launch_bounds__(MT_THREADS, (GATED && MT_N != 128) ? 1 : 2)
moe_grouped_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_w2,
                      const __grid_constant__ CUtensorMap map_a, void* __restrict__ out,
                      long long ldc, const int* __restrict__ tok, const int* __restrict__ c_index,
                      const float* __restrict__ c_scale, const int* __restrict__ tile_e, int N,
                      int K, int act) {
    pdl_launch_next();
    pdl_wait();                                    // the plan is the work of kernels before
    const int e = tile_e[blockIdx.y];
    if (e < 0) return;
    using TL = MTile<GATED, MT_N>;
    constexpr int MT_STAGES = TL::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + MT_STAGES * TL::STAGE_BYTES);
    uint64_t* empty = full + MT_STAGES;
    uint64_t* acc_full = empty + MT_STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* s_tok = (int*)(tmem_slot + 4);            // [MT_N] token of each row, -1: padding
    int* s_row = s_tok + MT_N;                     // [MT_N] output row
    float* s_scale = (float*)(s_row + MT_N);       // [MT_N]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * MT_M;              // first output feature
    const int n0 = blockIdx.y * MT_N;              // first sorted row
    const int n_kb = (K + MT_K - 1) / MT_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MT_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + MT_N) {
        const int i = threadIdx.x - 64, pos = n0 + i;
        s_tok[i] = tok[pos];
        s_row[i] = c_index ? c_index[pos] : pos;
        s_scale[i] = c_scale ? c_scale[pos] : 1.f;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)TL::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ loader
        const int wrow = e * N + m0;               // the expert's rows in the stacked matrix
        int issued = 0;
        for (int i = 0; i < n_kb; ++i) {
            const int s = i % MT_STAGES;
            const uint32_t ph = (i / MT_STAGES) & 1;
            if (*abort_flag) break;
            if (i >= MT_STAGES && !mbar_wait(&empty[s], ph ^ 1)) {
                atomicCAS(&g_moe_status, 0, (1 << 8) | s);
                *abort_flag = 1;
                break;
            }
            uint8_t* st = smem + s * TL::STAGE_BYTES;
            mbar_expect_tx(&full[s], TL::STAGE_BYTES);
            const int kx = i * MT_K;
            tma_load_2d(st, &map_w, kx, wrow, &full[s]);
            if (GATED) tma_load_2d(st + TL::A_BYTES, &map_w2, kx, wrow, &full[s]);
            tma_load_2d(st + TL::A_BYTES * (GATED ? 2 : 1), &map_a, kx, n0, &full[s]);
            ++issued;
        }
        if (*abort_flag) {
            // let the copies already issued land before the shared memory is given up
            const int first = issued > MT_STAGES ? issued - MT_STAGES : 0;
            for (int i = first; i < issued; ++i)
                mbar_wait(&full[i % MT_STAGES], (i / MT_STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ products
        constexpr uint32_t idesc = umma_idesc(MT_M, MT_N);
        bool ok = true;
        for (int i = 0; i < n_kb && ok; ++i) {
            const int s = i % MT_STAGES;
            const uint32_t ph = (i / MT_STAGES) & 1;
            if (*abort_flag) { ok = false; break; }
            if (!mbar_wait(&full[s], ph)) {
                atomicCAS(&g_moe_status, 0, (2 << 8) | s);
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(smem + s * TL::STAGE_BYTES);
            const uint32_t b_addr = a_addr + TL::A_BYTES * (GATED ? 2 : 1);
#pragma unroll
            for (int k = 0; k < MT_K / 16; ++k) {
                const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                const uint64_t bd = umma_desc(b_addr + k * 32);
                tc_mma_bf16(tmem_base, umma_desc(a_addr + k * 32), bd, idesc, acc);
                if (GATED)
                    tc_mma_bf16(tmem_base + MT_N, umma_desc(a_addr + TL::A_BYTES + k * 32), bd,
                                idesc, acc);
            }
            tc_commit(&empty[s]);          // the stage is free once these products have read it
        }
        tc_commit(acc_full);               // arrives when every product above is done
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;      // the tensor-memory lanes this warp may read
        bool ok = mbar_wait(acc_full, 0);
        if (!ok) {
            atomicCAS(&g_moe_status, 0, (3 << 8));
            *abort_flag = 1;
        }
        tc_fence_after();
        const bool run = ok && !*abort_flag;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // The tile goes through shared memory (the ring of stages is free once the
        // accumulator is complete) so that a row leaves in 16-byte pieces: [row][128 features].
        using TO = typename std::conditional<GATED, __nv_bfloat16, float>::type;
        static_assert(MT_N * MT_M * (int)sizeof(TO) <= MT_STAGES * TL::STAGE_BYTES,
                      "the output tile must fit the ring of stages");
        TO* ctile = (TO*)smem;
        const int fl = quarter * 32 + lane;
        if (run) {
#pragma unroll 1
            for (int c = 0; c < MT_N; c += 16) {
                uint32_t r[16], u[16];
                tc_ld16(lane_base + c, r);
                if (GATED) tc_ld16(lane_base + MT_N + c, u);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float v = __uint_as_float(r[j]);
                    if constexpr (GATED) {
                        v = mt_act(v, act) * __uint_as_float(u[j]);
                        ctile[(c + j) * MT_M + fl] = __float2bfloat16_rn(v);
                    } else {
                        ctile[(c + j) * MT_M + fl] = v * s_scale[c + j];
                    }
                }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps
        if (run) {
            constexpr int EPV = 16 / (int)sizeof(TO);          // elements per 16 bytes
            constexpr int VPR = MT_M / EPV;                    // 16-byte pieces per row
            const int et = (warp - 2) * 32 + lane;
            TO* obase = (TO*)out + m0;
            const bool fast = m0 + MT_M <= N && ldc % EPV == 0 && ((uintptr_t)obase & 15) == 0;
            if (fast) {
                for (int i = et; i < MT_N * VPR; i += 128) {
                    const int n = i / VPR, vi = i % VPR;
                    if (s_tok[n] < 0) continue;
                    *reinterpret_cast<uint4*>(obase + (size_t)s_row[n] * ldc + vi * EPV) =
                        reinterpret_cast<const uint4*>(ctile)[i];
                }
            } else {
                for (int i = et; i < MT_N * MT_M; i += 128) {
                    const int n = i / MT_M, f2 = i % MT_M;
                    if (s_tok[n] >= 0 && m0 + f2 < N) obase[(size_t)s_row[n] * ldc + f2] = ctile[i];
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)TL::TMEM_COLS)
                     : "memory");
    }
}

int mt_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld,
           int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return agv_fail(-4, "moe: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)MT_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return agv_fail(-4, "moe: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld, "
                        "ld %lld)", (int)r, rows, K, ld);
    return 0;
}

// xs[pos, :] = x[tok[pos], :] for the live rows of a plan, zeros for its padding.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                       const int* __restrict__ tok, __nv_bfloat16* __restrict__ xs, int rows,
                       int H) {
    pdl_wait();
    pdl_launch_next();
    const int per_row = H / 8;                         // 16-byte pieces of a row
    const long long total = (long long)rows * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / per_row), c = (int)(i % per_row);
        const int t = tok[pos];
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t >= 0) v = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + c * 8);
        *reinterpret_cast<uint4*>(xs + (size_t)pos * H + c * 8) = v;
    }
}

}  // namespace

// Whether the tensor-core grouped product takes these sizes (bfloat16 operands assumed).
AGV_API int agv_moe_grouped_tc_supported(int N, int K, long long lda) {
    return (N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0) ? 1 : 0;
}

// x: [T, H] bfloat16 rows of stride ldx; xs: [rows, H] dense.  H a multiple of 8, both
// 16-byte aligned.
AGV_API int agv_moe_gather_rows(const void* x, long long ldx, const int* tok, void* xs, int rows,
                                int H, cudaStream_t stream) {
    AGV_REQUIRE(rows >= 0 && H > 0 && H % 8 == 0 && ldx % 8 == 0, "moe_gather: rows of %d values "
                "with stride %lld do not move in 16-byte pieces", H, ldx);
    AGV_REQUIRE(agv_aligned(x, 16) && agv_aligned(xs, 16), "moe_gather: operands must be 16-byte "
                "aligned");
    if (rows == 0) return 0;
    long long blocks = ((long long)rows * (H / 8) + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    agv_launch(moe_gather_rows_kernel, (unsigned)blocks, 256, 0, stream, (const __nv_bfloat16*)x,
               ldx, tok, (__nv_bfloat16*)xs, rows, H);
    AGV_LAUNCH_OK("moe_gather_rows_kernel");
    return 0;
}

// a: [rows, K] bfloat16 in sorted order (row stride lda); w (and w2 for the gated form):
// [E, N, K] bfloat16 dense; tok, tile_e: the plan.  Gated: c [rows, N] bfloat16 rows of stride
// ldc at the sorted positions.  Plain: c 32-bit, row c_index[pos] (null: pos) times
// c_scale[pos] (null: 1).  tile: the plan's rows per tile, 64 or 128.
AGV_API int agv_moe_grouped_tc(const void* a, long long lda, int rows, const int* tok,
                               const void* w, const void* w2, int E, void* c, long long ldc,
                               const int* c_index, const float* c_scale, const int* tile_e,
                               int n_tiles, int tile, int N, int K, int act,
                               cudaStream_t stream) {
    AGV_REQUIRE(tile == 64 || tile == 128, "moe_grouped_tc: tiles of %d rows (64 or 128)", tile);
    AGV_REQUIRE(n_tiles >= 0 && E > 0 && rows >= n_tiles * tile, "moe_grouped_tc: bad sizes");
    AGV_REQUIRE(agv_moe_grouped_tc_supported(N, K, lda), "moe_grouped_tc: K (%d) and the row "
                "stride (%lld) must be multiples of 8", K, lda);
    AGV_REQUIRE(agv_aligned(a, 16) && agv_aligned(w, 16) && agv_aligned(w2, 16),
                "moe_grouped_tc: operands must be 16-byte aligned");
    AGV_REQUIRE(ldc >= N, "moe_grouped_tc: output row stride shorter than a row");
    AGV_REQUIRE((long long)E * N < (1ll << 31) && n_tiles <= 65535, "moe_grouped_tc: too large");
    if (n_tiles == 0) return 0;
    CUtensorMap mw, mw2, ma;
    if (int rc = mt_map(&mw, w, (long long)E * N, K, K, MT_M)) return rc;
    if (w2) {
        if (int rc = mt_map(&mw2, w2, (long long)E * N, K, K, MT_M)) return rc;
    } else {
        mw2 = mw;
    }
    if (int rc = mt_map(&ma, a, rows, K, lda, tile)) return rc;
    dim3 grid((N + MT_M - 1) / MT_M, n_tiles);
#define AGV_MT(GATED, BN)                                                                       \
    do {                                                                                        \
        auto kern = moe_grouped_tc_kernel<GATED, BN>;                                           \
        static bool configured = false;                                                         \
        if (!configured) {                                                                      \
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             MTile<GATED, BN>::SMEM));                          \
            configured = true;                                                                  \
        }                                                                                       \
        agv_launch(kern, grid, MT_THREADS, MTile<GATED, BN>::SMEM, stream, mw, mw2, ma, c, ldc, \
                   tok, c_index, c_scale, tile_e, N, K, act);                                   \
    } while (0)
    if (w2 && tile == 128) AGV_MT(true, 128);
    else if (w2) AGV_MT(true, 64);
    else if (tile == 128) AGV_MT(false, 128);
    else AGV_MT(false, 64);
#undef AGV_MT
    AGV_LAUNCH_OK("moe_grouped_tc_kernel");
    return 0;
}

// 0, or the code of the first bounded wait of the grouped kernel that gave up since the
// last call (the caller synchronises first).
AGV_API int agv_moe_tc_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_moe_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_moe_status, &zero, sizeof(int));
    }
    return v;
}
