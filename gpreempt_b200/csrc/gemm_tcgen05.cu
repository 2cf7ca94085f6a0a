// Preemptible bf16 GEMM on the 5th-generation tensor cores (tcgen05), the tensor-bound
// best-effort kernel of the preemption microbenchmark.
//
//   C[M][N] (bf16) = A[M][K] (bf16) x B[N][K]^T (bf16), fp32 accumulation in tensor memory.
//
// One persistent CTA per SM walks output tiles of 128 x 256 on a static schedule
// (tile = cta + iteration * grid).  Inside a CTA three roles run concurrently:
//   warp 0 (one lane)  TMA producer: streams 128x64 A and 256x64 B blocks (128-byte swizzle)
//                      through a 4-stage shared-memory ring and polls the preempt word,
//   warp 1 (one lane)  MMA issuer: four tcgen05.mma (128x256x16) per K block into TMEM,
//   warps 2-5          epilogue: tcgen05.ld the accumulator, convert to bf16, store C.
// The accumulator is double-buffered (2 x 256 of the 512 tensor-memory columns): while the
// epilogue drains one tile the MMA issuer already accumulates the next one in the other buffer.
//
// Preemption is K-block granular, not tile granular (a whole 128x256x8192 tile takes ~50 us,
// far above the 20 us drain target): when the producer sees the word raised it sends a STOP message
// down the ring; the MMA issuer commits what it has accumulated, the epilogue spills the fp32
// accumulator and the {iteration, K block} cursor of this CTA to the context buffer, and the
// CTA returns.  A relaunch with the same context reloads the accumulator into TMEM and
// continues with the next K block.  fp32 accumulators are saved exactly and the K order is
// unchanged, so the result is bit-identical to an uninterrupted run.  This is the K-granular
// form of the reference's tile-granular persistent loop
// (scripts/compile/convert_to_blp.py:39-70) and of BLPExecutor::resume
// (src/executor.cpp:280-298).
//
// Every wait is bounded; on a timeout the CTA records an error code in the context header,
// unwinds all roles, frees its tensor memory and returns.
#include "common.h"
#include "blp.cuh"
#include "sm100.cuh"

#include <cuda.h>
#include <cuda_bf16.h>

namespace gpx {

using namespace sm100;

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4, kUmmaK = 16;
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;  // two accumulator buffers of 256 columns
constexpr int kMaxGemmCtas = 256;
constexpr uint32_t kABytes = kBM * kBK * 2;           // 16 KiB
constexpr uint32_t kBBytes = kBN * kBK * 2;           // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;   // 48 KiB
constexpr size_t kGemmSmem = (size_t)kStages * kStageBytes + 1024 /*align*/ + 256 /*control*/;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s
constexpr int kPollEvery = 2;  // K blocks between polls of the preempt word

// Context buffer: header, one progress slot per CTA, one accumulator spill area per CTA.
struct GemmHeader {
    int error;       // 0 = none; otherwise role * 100 + site of the wait that gave up
    int error_cta;
    int pad[14];
};
struct GemmSlot {
    int next_iter;   // first iteration of this CTA's schedule that is not complete
    int k_done;      // K blocks already accumulated for that iteration (spill area is valid if > 0)
    int grid;        // grid size the schedule was started with (0 = fresh)
    int pad;
};
constexpr size_t kSlotOffset = sizeof(GemmHeader);
constexpr size_t kSpillOffset = 8192;
constexpr size_t kSpillBytesPerCta = (size_t)kBM * kBN * 4;
constexpr size_t kGemmCtxBytes = kSpillOffset + kMaxGemmCtas * kSpillBytesPerCta;
static_assert(kSlotOffset + kMaxGemmCtas * sizeof(GemmSlot) <= kSpillOffset, "slots overflow");

enum : int { MSG_DATA = 0, MSG_STOP = 1, MSG_EXIT = 2 };
enum : int { EPI_COMPLETE = 0, EPI_PARTIAL = 1, EPI_EXIT = 2 };

struct GemmControl {
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long tmem_full[2];   // one per accumulator buffer
    unsigned long long tmem_empty[2];
    uint32_t tmem_base;
    int stage_msg[kStages];
    int epi_kind[2];
    int epi_k_done[2];
    int epi_go;
    int abort_flag;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int &m_blk,
                                            int &n_blk) {
    // Groups of 16 row blocks sweep all column blocks, so tiles that run at the same time
    // share A and B panels in L2.
    constexpr int kGroup = 16;
    int group_size = kGroup * tiles_n;
    int group = tile / group_size;
    int first_m = group * kGroup;
    int rows = tiles_m - first_m < kGroup ? tiles_m - first_m : kGroup;
    int in_group = tile - group * group_size;
    m_blk = first_m + in_group % rows;
    n_blk = in_group / rows;
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, __nv_bfloat16 *C, int M, int N,
                         int K, unsigned char *ctx, BlpArgs blp) {
    extern __shared__ unsigned char smem_raw[];
    // Stage buffers need 1024-byte alignment for the 128-byte swizzle.
    uint32_t raw_addr = smem_u32(smem_raw);
    uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    unsigned char *smem = smem_raw + pad;
    GemmControl *ctl = reinterpret_cast<GemmControl *>(smem + (size_t)kStages * kStageBytes);
    const uint32_t smem_base = smem_u32(smem);
    volatile int *abort_flag = &ctl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = M / kBM, tiles_n = N / kBN;
    const int total_tiles = tiles_m * tiles_n;
    const int num_kb = K / kBK;

    GemmHeader *hdr = reinterpret_cast<GemmHeader *>(ctx);
    GemmSlot *slot = reinterpret_cast<GemmSlot *>(ctx + kSlotOffset) + blockIdx.x;
    float *spill = reinterpret_cast<float *>(ctx + kSpillOffset + (size_t)blockIdx.x * kSpillBytesPerCta);

    const int first_iter = slot->next_iter;
    const int first_k = slot->k_done;
    const int slot_grid = slot->grid;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl->tmem_full[b]), 2);   // tcgen05.commit + the issuer's own arrive
            mbar_init(smem_u32(&ctl->tmem_empty[b]), 1);
            ctl->epi_kind[b] = EPI_EXIT;
            ctl->epi_k_done[b] = 0;
        }
        ctl->abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        trace_begin(blp);
    }
    if (warp == 1) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl->tmem_base;

    // A schedule started with another grid size cannot be continued by this launch.
    const bool grid_ok = slot_grid == 0 || slot_grid == (int)gridDim.x;
    auto fail = [&](int code) {
        ctl->abort_flag = 1;
        if (atomicCAS(&hdr->error, 0, code) == 0) hdr->error_cta = blockIdx.x;
    };

    if (!grid_ok) {
        if (threadIdx.x == 0) fail(900);
    } else if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int flag = blp.preempted ? load_word(blp.preempted) : 0;
            int msg = MSG_EXIT;
            bool ok = true;
            for (int it = first_iter; ok; ++it) {
                int tile = blockIdx.x + it * gridDim.x;
                if (tile >= total_tiles) break;
                int m_blk, n_blk;
                tile_coords(tile, tiles_m, tiles_n, m_blk, n_blk);
                int kb0 = it == first_iter ? first_k : 0;
                for (int kb = kb0; kb < num_kb; ++kb) {
                    if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_flag, kWaitLimitNs)) {
                        fail(101);
                        ok = false;
                        break;
                    }
                    if (blp.preempted && ((kb - kb0) % kPollEvery) == 0) {
                        // The value tested was requested kPollEvery blocks ago, so the load's
                        // latency never stalls the ring.
                        if (flag != 0) {
                            msg = MSG_STOP;
                            ok = false;
                            break;
                        }
                        flag = load_word(blp.preempted);
                    }
                    ctl->stage_msg[stage] = MSG_DATA;
                    uint32_t bar = smem_u32(&ctl->full[stage]);
                    mbar_arrive_expect_tx(bar, kStageBytes);
                    uint32_t a_dst = smem_base + stage * kStageBytes;
                    tma_load_2d(a_dst, &tmap_a, bar, kb * kBK, m_blk * kBM);
                    tma_load_2d(a_dst + kABytes, &tmap_b, bar, kb * kBK, n_blk * kBN);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!*abort_flag) {
                // Terminal message (STOP after a raised word, EXIT when the schedule ran out).
                // For STOP the ring slot was already acquired above; for EXIT acquire it now.
                bool have_slot = msg == MSG_STOP;
                if (!have_slot)
                    have_slot = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_flag, kWaitLimitNs);
                if (have_slot) {
                    ctl->stage_msg[stage] = msg;
                    mbar_arrive(smem_u32(&ctl->full[stage]));
                } else {
                    fail(102);
                }
                if (msg == MSG_STOP && blp.trace) atomicMin(blp.trace + 2, globaltimer_ns());
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16_f32(kBM, kBN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t seg = 0;  // segments handed to the epilogue so far
            int it = first_iter;
            int kb = first_k;
            bool seg_open = false;  // tmem_empty already awaited for the current segment
            for (;;) {
                if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_flag, kWaitLimitNs)) {
                    fail(201);
                    break;
                }
                tc_fence_after_sync();
                int msg = ctl->stage_msg[stage];
                // Segments alternate between the two accumulator buffers, so the epilogue of one
                // tile runs while the next tile accumulates in the other buffer.
                const int buf = (int)(seg & 1);
                const uint32_t acc = tmem_base + buf * kBN;
                if (!seg_open) {
                    // The buffer is free (or restored) once the epilogue arrived for the segment
                    // that used it last; its completion number seg / 2 has parity (seg >> 1) & 1.
                    if (!mbar_wait(smem_u32(&ctl->tmem_empty[buf]), (seg >> 1) & 1, abort_flag, kWaitLimitNs)) {
                        fail(202);
                        break;
                    }
                    tc_fence_after_sync();
                    seg_open = true;
                }
                if (msg != MSG_DATA) {
                    ctl->epi_kind[buf] = msg == MSG_STOP ? EPI_PARTIAL : EPI_EXIT;
                    ctl->epi_k_done[buf] = kb;
                    mma_commit(smem_u32(&ctl->tmem_full[buf]));
                    mbar_arrive(smem_u32(&ctl->tmem_full[buf]));
                    break;
                }
                uint32_t a_addr = smem_base + stage * kStageBytes;
                uint64_t a_desc = make_smem_desc_sw128(a_addr);
                uint64_t b_desc = make_smem_desc_sw128(a_addr + kABytes);
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k) {
                    // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in the
                    // descriptor's 16-byte address units.
                    mma_f16_ss(acc, a_desc + 2 * k, b_desc + 2 * k, idesc,
                               (kb > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(smem_u32(&ctl->empty[stage]));  // ring slot reusable once these retire
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
                if (++kb == num_kb) {
                    ctl->epi_kind[buf] = EPI_COMPLETE;
                    ctl->epi_k_done[buf] = num_kb;
                    mma_commit(smem_u32(&ctl->tmem_full[buf]));
                    mbar_arrive(smem_u32(&ctl->tmem_full[buf]));
                    ++seg;
                    ++it;
                    kb = 0;
                    seg_open = false;
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (4 warps)
        const int quarter = warp & 3;                 // TMEM lanes this warp may access
        const int row = quarter * 32 + lane;          // accumulator row == TMEM lane
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const bool leader = threadIdx.x == 64;
        uint32_t v[32];
        if (first_k > 0) {
            // Resume: reload the spilled fp32 accumulator into tensor memory.
            for (int c = 0; c < kBN; c += 32) {
                // (layout of the spill area: see the store below)
                const uint4 *src = reinterpret_cast<const uint4 *>(spill) + (size_t)(c / 32) * 8 * 128 + row;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint4 q = src[j * 128];
                    v[4 * j + 0] = q.x;
                    v[4 * j + 1] = q.y;
                    v[4 * j + 2] = q.z;
                    v[4 * j + 3] = q.w;
                }
                tmem_st_32x32(t_lane + c, v);
            }
            tmem_st_wait();
        }
        tc_fence_before_sync();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (leader) {
            mbar_arrive(smem_u32(&ctl->tmem_empty[0]));  // a restored tile sits in buffer 0: segment 0 uses it
            mbar_arrive(smem_u32(&ctl->tmem_empty[1]));
        }

        int it = first_iter;
        int seg_k0 = first_k;
        int tiles_done = 0;
        for (uint32_t seg = 0;; ++seg) {
            const int buf = (int)(seg & 1);
            const uint32_t t_acc = t_lane + buf * kBN;
            // One thread waits on the mbarrier and publishes the outcome, so the 128 epilogue
            // threads always take the same branch and never strand one another at bar.sync.
            if (leader) {
                bool ok = mbar_wait(smem_u32(&ctl->tmem_full[buf]), (seg >> 1) & 1, abort_flag, kWaitLimitNs);
                if (!ok) fail(301);
                ctl->epi_go = ok ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!ctl->epi_go) break;
            tc_fence_after_sync();
            const int kind = ctl->epi_kind[buf];
            const int k_done = ctl->epi_k_done[buf];
            if (kind == EPI_EXIT) {
                if (leader) {
                    slot->next_iter = it;
                    slot->k_done = 0;
                    slot->grid = gridDim.x;
                }
                break;
            }
            if (kind == EPI_COMPLETE) {
                int tile = blockIdx.x + it * gridDim.x;
                int m_blk, n_blk;
                tile_coords(tile, tiles_m, tiles_n, m_blk, n_blk);
                __nv_bfloat16 *crow = C + (size_t)(m_blk * kBM + row) * N + (size_t)n_blk * kBN;
                for (int c = 0; c < kBN; c += 32) {
                    tmem_ld_32x32(t_acc + c, v);
                    tmem_ld_wait();
                    uint4 *dst = reinterpret_cast<uint4 *>(crow + c);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 q;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 0]),
                                                                  __uint_as_float(v[8 * j + 1]));
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2]),
                                                                  __uint_as_float(v[8 * j + 3]));
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 4]),
                                                                  __uint_as_float(v[8 * j + 5]));
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 6]),
                                                                  __uint_as_float(v[8 * j + 7]));
                        q.x = *reinterpret_cast<uint32_t *>(&p0);
                        q.y = *reinterpret_cast<uint32_t *>(&p1);
                        q.z = *reinterpret_cast<uint32_t *>(&p2);
                        q.w = *reinterpret_cast<uint32_t *>(&p3);
                        dst[j] = q;
                    }
                }
                ++it;
                ++tiles_done;
                seg_k0 = 0;
                // Hand the accumulator back to the MMA issuer.
                tc_fence_before_sync();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (leader) {
                    mbar_arrive(smem_u32(&ctl->tmem_empty[buf]));
                    if (blp.executed) atomicAdd(blp.executed, 1);
                }
                continue;
            }
            // EPI_PARTIAL: spill the accumulator if this launch added to it, record the cursor.
            if (k_done > seg_k0) {
                for (int c = 0; c < kBN; c += 32) {
                    tmem_ld_32x32(t_acc + c, v);
                    tmem_ld_wait();
                    // The spill area is private to this kernel, so its layout is chosen for the
                    // stores: the j-th 16-byte piece of a 32-column chunk of all 128 rows is
                    // contiguous and one warp store writes 512 consecutive bytes (with row-major
                    // rows, 1 KB apart, every thread of a store touched its own line).
                    uint4 *dst = reinterpret_cast<uint4 *>(spill) + (size_t)(c / 32) * 8 * 128 + row;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        dst[j * 128] = make_uint4(v[4 * j + 0], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
            if (leader) {
                slot->next_iter = it;
                slot->k_done = k_done;
                slot->grid = gridDim.x;
                if (blp.stop_index) atomicCAS(blp.stop_index, -1, blp.kernel_id);
            }
            break;
        }
        if (leader && blp.trace && tiles_done)
            atomicAdd(blp.trace + 3, (unsigned long long)tiles_done);
    }

    // All roles meet here; tensor memory is released by the warp that allocated it.
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0 && lane == 0 && *abort_flag) {
        // Error path: give loads that are still in flight a bounded chance to land before the
        // CTA's shared memory is handed to another CTA.
        for (int spin = 0; spin < 64; ++spin) __nanosleep(1000);
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && blp.trace) atomicMax(blp.trace + 1, globaltimer_ns());
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tmap_2d_bf16(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols,
                      uint32_t box_rows, uint32_t box_cols) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) encode = reinterpret_cast<EncodeTiledFn>(driver_entry("cuTensorMapEncodeTiled"));
    GPX_REQUIRE(encode, GPX_FAIL, "driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    GPX_REQUIRE(rc == CUDA_SUCCESS, GPX_FAIL, "cuTensorMapEncodeTiled failed with %d", (int)rc);
    return GPX_SUCC;
}

}  // namespace gpx

using namespace gpx;

extern "C" {

int gpx_gemm_ctx_bytes(size_t *bytes) {
    GPX_REQUIRE(bytes, GPX_FAIL, "bytes is NULL");
    *bytes = kGemmCtxBytes;
    return GPX_SUCC;
}

int gpx_gemm_tiles(int M, int N, int *tiles) {
    GPX_REQUIRE(tiles, GPX_FAIL, "tiles is NULL");
    GPX_REQUIRE(M > 0 && N > 0 && M % kBM == 0 && N % kBN == 0, GPX_OUT_OF_RANGE,
                "M must be a multiple of %d and N of %d", kBM, kBN);
    *tiles = (M / kBM) * (N / kBN);
    return GPX_SUCC;
}

int gpx_gemm_status(const void *ctx, int *error, int *error_cta) {
    GPX_REQUIRE(ctx && error, GPX_FAIL, "NULL argument");
    GemmHeader h;
    GPX_CUDA(cudaMemcpy(&h, ctx, sizeof(h), cudaMemcpyDeviceToHost));
    *error = h.error;
    if (error_cta) *error_cta = h.error_cta;
    return GPX_SUCC;
}

int gpx_gemm_bf16(const void *A, const void *B, void *C, int M, int N, int K, void *ctx,
                  const gpx_blp *blp, gpx_stream s) {
    GPX_REQUIRE(A && B && C && ctx, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(M > 0 && N > 0 && K > 0 && M % kBM == 0 && N % kBN == 0 && K % kBK == 0,
                GPX_OUT_OF_RANGE, "M, N, K must be multiples of %d, %d, %d", kBM, kBN, kBK);
    GPX_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)B % 16) == 0 && ((uintptr_t)C % 16) == 0 &&
                    ((uintptr_t)ctx % 16) == 0,
                GPX_FAIL, "A, B, C and ctx must be 16-byte aligned");
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    CUtensorMap ta, tb;
    GPX_TRY(make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, kBM, kBK));
    GPX_TRY(make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, kBN, kBK));
    static bool attr_set[64] = {false};
    if (!attr_set[d.device]) {
        GPX_CUDA(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem));
        attr_set[d.device] = true;
    }
    BlpArgs b{};
    int tiles = (M / kBM) * (N / kBN);
    b.total_tiles = tiles;
    if (blp) {
        b.preempted = (const int *)blp->preempted;
        b.stop_index = (int *)blp->stop_index;
        b.executed = (int *)blp->executed;
        b.kernel_id = blp->kernel_id;
        b.trace = (unsigned long long *)blp->trace;
        GPX_REQUIRE(!b.preempted || b.stop_index, GPX_FAIL, "preemptible launch needs stop_index");
    }
    int grid = d.sm_count < kMaxGemmCtas ? d.sm_count : kMaxGemmCtas;
    if (grid > tiles) grid = tiles;
    gemm_bf16_tcgen05_kernel<<<grid, kGemmThreads, kGemmSmem, as_stream(s)>>>(
        ta, tb, (__nv_bfloat16 *)C, M, N, K, (unsigned char *)ctx, b);
    GPX_CUDA(cudaGetLastError());
    return GPX_SUCC;
}

}  // extern "C"

// ---- variant that allocates nothing ------------------------------------------------------------
//
// Some callers of this GEMM cannot allocate device memory: a client whose device memory is
// handed out once by an external pool or a memory-capped container, a latency-critical thread
// that must not enter the allocator (cudaMalloc can synchronise the whole device), or code that
// runs where allocation is simply not permitted.  For them the progress slots and the
// accumulator spill area live in the file-scope array below instead of a caller-allocated
// context.  The array is sized for kStaticMaxTiles output tiles (one CTA per tile), is part of
// the library image and is held by every GPU that loads the library until the process exits.
namespace gpx {

constexpr int kStaticMaxTiles = 64;
constexpr size_t kStaticCtxBytes = kSpillOffset + (size_t)kStaticMaxTiles * kSpillBytesPerCta;

static __device__ __align__(256) unsigned char g_gemm_static_ctx[kStaticCtxBytes];

// Device address of g_gemm_static_ctx on each device.  In host code the array's name is only a
// host-side stand-in for the symbol, never a device address, so the address is looked up once
// per device (with that device current) and cached.
static unsigned char *g_static_ctx_addr[64] = {nullptr};

static int static_ctx_address(int device, unsigned char **out) {
    // cudaGetSymbolAddress answers for the device that is current in the CUDA runtime, which is
    // not necessarily the one this thread bound with gpx_init (another library may have called
    // cudaSetDevice since): a pointer cached under the wrong index would send every later call on
    // that device to another GPU's array.
    int current = -1;
    cudaError_t err = cudaGetDevice(&current);
    if (err != cudaSuccess || current != device || device < 0 || device >= 64) {
        set_error("gpx_gemm_bf16_static: the CUDA current device is %d but this thread was bound to device %d "
                  "by gpx_init; make device %d current (or call gpx_init again) before the call",
                  current, device, device);
        return GPX_FAIL;
    }
    if (!g_static_ctx_addr[device]) {
        void *p = nullptr;
        err = cudaGetSymbolAddress(&p, g_gemm_static_ctx);
        if (err != cudaSuccess || !p) {
            set_error("cudaGetSymbolAddress(g_gemm_static_ctx) failed on device %d: %s", device,
                      cudaGetErrorString(err));
            return GPX_FAIL;
        }
        g_static_ctx_addr[device] = (unsigned char *)p;
    }
    *out = g_static_ctx_addr[device];
    return GPX_SUCC;
}

}  // namespace gpx

extern "C" int gpx_gemm_bf16_static(const void *A, const void *B, void *C, int M, int N, int K,
                                    int resume, const gpx_blp *blp, gpx_stream s) {
    GPX_REQUIRE(A && B && C, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(M > 0 && N > 0 && K > 0 && M % kBM == 0 && N % kBN == 0 && K % kBK == 0,
                GPX_OUT_OF_RANGE, "M, N, K must be multiples of %d, %d, %d", kBM, kBN, kBK);
    GPX_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)B % 16) == 0 && ((uintptr_t)C % 16) == 0,
                GPX_FAIL, "A, B and C must be 16-byte aligned");
    const int tiles = (M / kBM) * (N / kBN);
    GPX_REQUIRE(tiles <= kStaticMaxTiles, GPX_OUT_OF_RANGE,
                "gpx_gemm_bf16_static handles at most %d output tiles of %dx%d (M/%d * N/%d = %d "
                "here); use gpx_gemm_bf16 with a caller-allocated context for larger products",
                kStaticMaxTiles, kBM, kBN, kBM, kBN, tiles);
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    unsigned char *ctx = nullptr;
    GPX_TRY(static_ctx_address(d.device, &ctx));
    CUtensorMap ta, tb;
    GPX_TRY(make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, kBM, kBK));
    GPX_TRY(make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, kBN, kBK));
    static bool attr_set[64] = {false};
    if (!attr_set[d.device]) {
        GPX_CUDA(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem));
        attr_set[d.device] = true;
    }
    BlpArgs b{};
    b.total_tiles = tiles;
    if (blp) {
        b.preempted = (const int *)blp->preempted;
        b.stop_index = (int *)blp->stop_index;
        b.executed = (int *)blp->executed;
        b.kernel_id = blp->kernel_id;
        b.trace = (unsigned long long *)blp->trace;
        GPX_REQUIRE(!b.preempted || b.stop_index, GPX_FAIL, "preemptible launch needs stop_index");
    }
    // The array keeps the previous call's contents.  A fresh product must start from zeroed
    // progress slots and error header; a resume must find them as the drained launch left them.
    if (!resume) GPX_CUDA(cudaMemsetAsync(ctx, 0, kSpillOffset, as_stream(s)));
    int grid = tiles < d.sm_count ? tiles : d.sm_count;
    gemm_bf16_tcgen05_kernel<<<grid, kGemmThreads, kGemmSmem, as_stream(s)>>>(
        ta, tb, (__nv_bfloat16 *)C, M, N, K, ctx, b);
    GPX_CUDA(cudaGetLastError());
    return GPX_SUCC;
}

extern "C" int gpx_gemm_static_status(int *error, int *error_cta) {
    GPX_REQUIRE(error, GPX_FAIL, "NULL argument");
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    unsigned char *ctx = nullptr;
    GPX_TRY(static_ctx_address(d.device, &ctx));
    GemmHeader h;
    GPX_CUDA(cudaMemcpy(&h, ctx, sizeof(h), cudaMemcpyDeviceToHost));
    *error = h.error;
    if (error_cta) *error_cta = h.error_cta;
    return GPX_SUCC;
}
