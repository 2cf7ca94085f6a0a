// Convolution as a row-shifted GEMM on the tcgen05 tensor cores, fp32 accuracy from split-bf16
// operands, K-block-granular preemption.
//
// Stands in for the TVM-generated fused conv2d(+bias)(+add)(+relu) kernels the reference
// replays (src/executor.cpp:157-162).  Activations and weights are stored as two bf16 planes
// (x ~= hi + lo); one fp32 product is three tensor-core products hi*hi + hi*lo + lo*hi
// accumulated in fp32 in tensor memory, which keeps 16 mantissa bits per operand and meets the
// 1e-4 parity bound of the fp32 configuration at a third of the bf16 tensor rate.
//
// GEMM view: rows are stored pixels of the input (see act_layout.h), a filter tap is a constant
// row shift, so the A operand of every K block is a plain 2-D TMA tile [128 rows][64 channels]
// at row (m0 + shift[tap]); rows outside the tensor are zero-filled by TMA.  B is the weight
// matrix [Cout][taps*Cin].  Rows that are not real output pixels (image borders of the padded
// layouts) are computed and dropped by the epilogue.
//
// Single-plane models (bf16 / fp16 storage) use the same kernel with one product per K step and
// twice as many ring stages.
//
// CTA roles, ring, messages and the preempt / spill / resume protocol are those of
// gemm_tcgen05.cu, with two accumulator buffers in tensor memory so that the epilogue of one
// tile overlaps the K loop of the next.  The epilogue adds the bias, applies the activation,
// splits the fp32 result into the plane format and writes each row into the consumer's layout
// with 256-bit stores.  The residual of a 1x1 convolution on plain rows is added by the tensor
// core itself: extra K blocks whose A operand is the residual tile and whose B operand is a
// 64x64 identity tile kept in shared memory; other residuals are added by the epilogue.
#include "layers.cuh"
#include "sm100.cuh"

#include <cuda_bf16.h>

namespace gpx {

using namespace sm100;

constexpr int kCBM = 128, kCBK = 64, kCUmmaK = 16;
// Warp 0 feeds TMA, warp 1 issues MMAs, the other warps are the epilogue: kCEpiParts warps per
// TMEM lane quarter, each taking an equal share of the columns in 16-column pieces, so that
// enough independent TMEM loads, conversions and stores are in flight while a tile is drained
// (the epilogue, not the tensor pipe, bounds the small-K layers).
constexpr int kCEpiParts = 2;                       // epilogue warps per TMEM lane quarter
constexpr int kCEpiThreads = 128 * kCEpiParts;
constexpr int kCgemmThreads = 64 + kCEpiThreads;
constexpr unsigned long long kCWaitLimitNs = 2000000000ull;
constexpr int kCPollEvery = 1;

struct CgemmControlSize {
    unsigned char bytes[2560];  // room for CgemmControl (checked below)
};

template <int BN>
struct CgemmCfg {
    static constexpr uint32_t kABytes = kCBM * kCBK * 2;        // one plane of A: 16 KiB
    static constexpr uint32_t kWBytes = BN * kCBK * 2;          // one plane of W
    static constexpr uint32_t kStageBytes = 2 * kABytes + 2 * kWBytes;
    static constexpr int kStages = BN == 256 ? 2 : (BN == 128 ? 3 : 4);
    // ring + alignment slack + 64x64 identity tile + control block
    static constexpr uint32_t kIdentBytes = 64 * kCBK * 2;
    static constexpr size_t kSmem =
        (size_t)kStages * kStageBytes + 1024 + kIdentBytes + sizeof(CgemmControlSize);
    // Four fp32 accumulators per tile (see the MMA issuer): hi*hi of even K steps, hi*hi of odd
    // K steps, hi*lo, lo*hi.  256 or 512 TMEM columns, both powers of two.
    // (256-column tiles exist for the two-accumulator plan only: 2 x 256 columns, one buffer.)
    static constexpr int kAccs = BN == 256 ? 2 : 4;
    static constexpr int kTmemCols = kAccs * BN;
};

enum : int { CMSG_DATA = 0, CMSG_STOP = 1, CMSG_EXIT = 2, CMSG_RES = 3 };
enum : int { CEPI_COMPLETE = 0, CEPI_PARTIAL = 1, CEPI_EXIT = 2 };

struct CgemmControl {
    unsigned long long full[8];
    unsigned long long empty[8];
    unsigned long long tmem_full[2];   // one per accumulator buffer
    unsigned long long tmem_empty[2];
    uint32_t tmem_base;
    int stage_msg[8];
    int epi_kind[2];
    int epi_k_done[2];
    int epi_go;
    int raised;  // the word was up when this CTA started
    int abort_flag;
    float bias_s[2][256];  // bias of the tile each accumulator buffer holds, staged by the epilogue
};

static_assert(sizeof(CgemmControl) <= sizeof(CgemmControlSize), "control block outgrew its shared-memory budget");

// x / d for 0 <= x < 2^24 and d > 0 with `inv` = 1.0f / d: the float quotient is off by at most
// one, which the remainder corrects.  An integer division by a run-time divisor is a chain of
// ~30 dependent instructions; the epilogue decodes its tile and its row with six of them, about a
// microsecond per tile for a lone warp, which is what bounded the layers with one or two K blocks.
__device__ __forceinline__ int fast_div(int x, int d, float inv) {
    int q = (int)((float)x * inv);
    int r = x - q * d;
    if (r < 0) --q;
    if (r >= d) ++q;
    return q;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&p);
}
// Pulls a TMA descriptor (kernel parameter) into the descriptor cache ahead of its first use.
__device__ __forceinline__ void prefetch_tensormap(const void *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// 256-bit global accesses (32-byte aligned): one whole sector per lane.
__device__ __forceinline__ void ld_global_v8(const void *ptr, uint32_t *r) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(ptr));
}
__device__ __forceinline__ void st_global_v8(void *ptr, const uint32_t *r) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ float bf16_lo_to_f32(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi_to_f32(uint32_t packed) {
    return __uint_as_float(packed & 0xffff0000u);
}

// Phase timers of a development build (-DGPX_CGEMM_TIMING): clock64 deltas summed over CTAs into a
// device array that gpx_debug_cgemm_timing reads.  Compiled out otherwise.
#ifdef GPX_CGEMM_TIMING
__device__ unsigned long long g_cgemm_timing[32];
#define TCK(var) long long var = clock64()
#define TADD(slot, val) atomicAdd(&g_cgemm_timing[slot], (unsigned long long)(val))
#else
#define TCK(var)
#define TADD(slot, val)
#endif

template <int BN>
__global__ void __launch_bounds__(kCgemmThreads, 1)
cgemm_tcgen05_kernel(const __grid_constant__ CgemmParams p, BlpArgs blp) {
    using Cfg = CgemmCfg<BN>;
    constexpr int kStages = Cfg::kStages;
    TCK(t_start);
    // The prologue below (barriers, tensor memory, descriptor prefetch) touches nothing a
    // predecessor kernel writes, so it runs while that kernel drains; pdl_wait() comes after it.
    extern __shared__ unsigned char smem_raw[];
    uint32_t raw_addr = smem_u32(smem_raw);
    uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    unsigned char *smem = smem_raw + pad;
    // The identity tile follows the ring (1024-byte aligned, as its swizzled layout needs).
    const uint32_t ident_off = kStages * Cfg::kStageBytes;
    CgemmControl *ctl = reinterpret_cast<CgemmControl *>(smem + ident_off + Cfg::kIdentBytes);
    const uint32_t smem_base = smem_u32(smem);
    volatile int *abort_flag = &ctl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // A tile is (row block, column block, K split); splits of one output block are adjacent so
    // they run at the same time.  With k_splits == 1 a tile covers the whole K range.
    const int total_tiles = p.tiles_m * p.tiles_n * p.k_splits;
    const int all_kb = p.taps * p.cin_blocks;
    auto tile_kb_begin = [&](int tile) { return (tile % p.k_splits) * p.kb_per_split; };
    auto tile_kb_count = [&](int tile) {
        int left = all_kb - (tile % p.k_splits) * p.kb_per_split;
        return left < p.kb_per_split ? left : p.kb_per_split;
    };
    const bool resumable = blp.preempted != nullptr;
    // Two-plane operands (float32 models) or one 16-bit plane (reduced-precision models).
    const bool two_plane = p.fmt == PF_SPLIT;
    // A ring stage holds the A and W tiles of one K block: hi and lo planes of both for float32
    // models; single-plane models use half of that per stage and get twice as many stages, which
    // doubles the bytes TMA keeps in flight.
    const int nst = two_plane ? kStages : 2 * kStages;
    const uint32_t stage_bytes = two_plane ? Cfg::kStageBytes : Cfg::kStageBytes / 2;
    const uint32_t w_off = two_plane ? 2 * Cfg::kABytes : Cfg::kABytes;  // W (hi) tile inside a stage
    // Accumulator plan.  dual: two accumulators per tile (BN columns each) in two buffers, so the
    // epilogue of one tile overlaps the K loop of the next; used when the K range is short or the
    // operands are single-plane.  Otherwise four accumulators in one buffer (see the MMA issuer).
    const bool dual = p.dual != 0;
    const int nbuf = (dual && 4 * BN <= 512) ? 2 : 1;
    const int buf_cols = dual ? 2 * BN : Cfg::kTmemCols;

    CgemmSlot *slot = p.slots + blockIdx.x;
    float *spill = p.spill + (size_t)blockIdx.x * (kCBM * Cfg::kTmemCols);

    if (threadIdx.x == 0) {
        for (int s = 0; s < nst; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl->tmem_full[b]), 2);
            mbar_init(smem_u32(&ctl->tmem_empty[b]), 1);
            ctl->epi_kind[b] = CEPI_EXIT;
            ctl->epi_k_done[b] = 0;
        }
        ctl->abort_flag = 0;
        ctl->epi_go = 0;
        ctl->raised = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&p.a_hi);
        prefetch_tensormap(&p.w_hi);
        if (two_plane) {
            prefetch_tensormap(&p.a_lo);
            prefetch_tensormap(&p.w_lo);
        }
    }
    if (warp == 1) tmem_alloc(smem_u32(&ctl->tmem_base), Cfg::kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl->tmem_base;

    // A non-preemptible launch knows its first tile without reading the cursor, and weights are
    // never written by a kernel: its producer thread fetches the weight tiles of the first ring
    // stages before it waits for the predecessor, so that their latency overlaps the
    // predecessor's tail (batch-1 forwards are chains of such latencies).  Every other thread,
    // and every thread of a preemptible launch, waits here.
    const bool early_weights = !resumable && (int)blockIdx.x < total_tiles;
    int prearmed = 0;  // ring stages whose barrier is armed and whose weight loads are in flight
    if (early_weights && threadIdx.x == 0) {
        const int tile = blockIdx.x;
        const int n_blk = (tile / p.k_splits) % p.tiles_n;
        const int main_kb = tile_kb_count(tile);
        const int kb_base = tile_kb_begin(tile);
        uint32_t ident_bytes = p.res_kb ? Cfg::kIdentBytes : 0u;
        for (int kb = 0; kb < main_kb && kb < nst; ++kb) {
            const int tap = (kb_base + kb) / p.cin_blocks;
            const int cb = (kb_base + kb) - tap * p.cin_blocks;
            const uint32_t bar = smem_u32(&ctl->full[kb]);
            ctl->stage_msg[kb] = CMSG_DATA;
            mbar_arrive_expect_tx(bar, (two_plane ? Cfg::kStageBytes : Cfg::kABytes + Cfg::kWBytes) + ident_bytes);
            if (ident_bytes) tma_load_2d(smem_base + ident_off, &p.ident, bar, 0, 0);
            ident_bytes = 0;
            const uint32_t dst = smem_base + kb * stage_bytes;
            const int w_col = tap * p.cin + cb * kCBK;
            tma_load_2d(dst + w_off, &p.w_hi, bar, w_col, n_blk * BN);
            if (two_plane) tma_load_2d(dst + 2 * Cfg::kABytes + Cfg::kWBytes, &p.w_lo, bar, w_col, n_blk * BN);
            ++prearmed;
        }
    }
    pdl_wait();  // from here on the predecessor's results (and this executor's slots) are visible
    pdl_launch_dependents();

    // A non-preemptible launch never stops early, so it neither reads nor writes the cursor.
    const int first_iter = resumable ? slot->next_iter : 0;
    const int first_k = resumable ? slot->k_done : 0;
    const int slot_grid = resumable ? slot->grid : 0;

    // A kernel that starts while the word is raised (it was queued behind the stop point) leaves
    // at once: the cursor is unchanged, the stop point is recorded if this CTA still has work
    // (kernel_transform_be.py:10-12).
    if (resumable) {
        if (threadIdx.x == 0) {
            const int raised = load_word(blp.preempted);
            if (raised) {
                if ((int)blockIdx.x + first_iter * (int)gridDim.x < total_tiles && blp.stop_index)
                    atomicCAS(blp.stop_index, -1, blp.kernel_id);
                if (blp.trace) {
                    unsigned long long t = globaltimer_ns();
                    atomicMin(blp.trace + 0, t);
                    atomicMin(blp.trace + 2, t);
                    atomicMax(blp.trace + 1, t);
                }
            }
            ctl->raised = raised;
        }
        tc_fence_before_sync();
        __syncthreads();
        if (ctl->raised) {
            if (warp == 1) {
                tc_fence_after_sync();
                tmem_dealloc(tmem_base, Cfg::kTmemCols);
            }
            return;
        }
    }
    if (threadIdx.x == 0) trace_begin(blp);
#ifdef GPX_CGEMM_TIMING
    if (threadIdx.x == 0) TADD(14, clock64() - t_start);
#endif

    const bool grid_ok = slot_grid == 0 || slot_grid == (int)gridDim.x;
    auto fail = [&](int code) {
        ctl->abort_flag = 1;
        if (atomicCAS(p.error, 0, code) == 0) p.error[1] = blp.kernel_id * 1000 + (int)blockIdx.x;
    };

    if (!grid_ok) {
        if (threadIdx.x == 0) fail(900);
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int flag = resumable ? load_word(blp.preempted) : 0;
            int msg = CMSG_EXIT;
            bool ok = true;
            // The identity tile travels with the first stage this CTA fills.
            uint32_t ident_bytes = (p.res_kb && prearmed == 0) ? Cfg::kIdentBytes : 0u;
            TCK(t_prod0);
#ifdef GPX_CGEMM_TIMING
            long long prod_wait = 0;
#endif
            for (int it = first_iter; ok; ++it) {
                int tile = blockIdx.x + it * gridDim.x;
                if (tile >= total_tiles) break;
                // Column tiles vary fastest: CTAs that run together share the same A rows.
                const int n_blk = (tile / p.k_splits) % p.tiles_n;
                const int m_blk = (tile / p.k_splits) / p.tiles_n;
                const int kb0 = it == first_iter ? first_k : 0;
                const int main_kb = tile_kb_count(tile);
                const int num_kb = main_kb + p.res_kb;  // the residual rides along as extra K blocks
                const int kb_base = tile_kb_begin(tile);
                for (int kb = kb0; kb < num_kb; ++kb) {
                    TCK(t_w0);
                    if (it == first_iter && kb < prearmed) {
                        // armed before the wait for the predecessor, weights already on their way:
                        // only the activation tiles are missing
                        const int tap = (kb_base + kb) / p.cin_blocks;
                        const int cb = (kb_base + kb) - tap * p.cin_blocks;
                        const uint32_t bar = smem_u32(&ctl->full[stage]);
                        const uint32_t dst = smem_base + stage * stage_bytes;
                        const int a_row = m_blk * kCBM + p.tap_shift[tap];
                        tma_load_2d(dst, &p.a_hi, bar, cb * kCBK, a_row);
                        if (two_plane) tma_load_2d(dst + Cfg::kABytes, &p.a_lo, bar, cb * kCBK, a_row);
                        if (++stage == nst) {
                            stage = 0;
                            phase ^= 1;
                        }
                        continue;
                    }
                    if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_flag, kCWaitLimitNs)) {
                        fail(101);
                        ok = false;
                        break;
                    }
#ifdef GPX_CGEMM_TIMING
                    prod_wait += clock64() - t_w0;
#endif
                    if (resumable && ((kb - kb0) % kCPollEvery) == 0) {
                        if (flag != 0) {
                            msg = CMSG_STOP;
                            ok = false;
                            break;
                        }
                        flag = load_word(blp.preempted);
                    }
                    const uint32_t bar = smem_u32(&ctl->full[stage]);
                    if (kb >= main_kb) {
                        // Residual block: A = 64 channels of the residual rows of this tile; the W
                        // operand is the 64x64 identity that stays in shared memory, applied to the
                        // matching 64 accumulator columns, so the tensor core adds the residual.
                        const int rb = kb - main_kb;
                        ctl->stage_msg[stage] = CMSG_RES + rb;
                        mbar_arrive_expect_tx(bar, (two_plane ? 2 : 1) * Cfg::kABytes + ident_bytes);
                        const uint32_t dst = smem_base + stage * stage_bytes;
                        tma_load_2d(dst, &p.r_hi, bar, n_blk * BN + rb * kCBK, m_blk * kCBM);
                        if (two_plane) tma_load_2d(dst + Cfg::kABytes, &p.r_lo, bar, n_blk * BN + rb * kCBK, m_blk * kCBM);
                        if (ident_bytes) tma_load_2d(smem_base + ident_off, &p.ident, bar, 0, 0);
                        ident_bytes = 0;
                        if (++stage == nst) {
                            stage = 0;
                            phase ^= 1;
                        }
                        continue;
                    }
                    const int tap = (kb_base + kb) / p.cin_blocks;
                    const int cb = (kb_base + kb) - tap * p.cin_blocks;
                    ctl->stage_msg[stage] = CMSG_DATA;
                    mbar_arrive_expect_tx(bar, (two_plane ? Cfg::kStageBytes : Cfg::kABytes + Cfg::kWBytes) + ident_bytes);
                    if (ident_bytes) tma_load_2d(smem_base + ident_off, &p.ident, bar, 0, 0);
                    ident_bytes = 0;
                    const uint32_t dst = smem_base + stage * stage_bytes;
                    const int a_row = m_blk * kCBM + p.tap_shift[tap];
                    const int w_col = tap * p.cin + cb * kCBK;
                    tma_load_2d(dst, &p.a_hi, bar, cb * kCBK, a_row);
                    tma_load_2d(dst + w_off, &p.w_hi, bar, w_col, n_blk * BN);
                    if (two_plane) {
                        tma_load_2d(dst + Cfg::kABytes, &p.a_lo, bar, cb * kCBK, a_row);
                        tma_load_2d(dst + 2 * Cfg::kABytes + Cfg::kWBytes, &p.w_lo, bar, w_col, n_blk * BN);
                    }
                    if (++stage == nst) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
#ifdef GPX_CGEMM_TIMING
            TADD(0, prod_wait);
            TADD(1, clock64() - t_prod0);
#endif
            if (!*abort_flag) {
                bool have_slot = msg == CMSG_STOP;
                if (!have_slot)
                    have_slot = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1, abort_flag, kCWaitLimitNs);
                if (have_slot) {
                    ctl->stage_msg[stage] = msg;
                    mbar_arrive(smem_u32(&ctl->full[stage]));
                } else {
                    fail(102);
                }
                if (msg == CMSG_STOP && blp.trace) atomicMin(blp.trace + 2, globaltimer_ns());
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        // The whole warp walks the K loop in lock step and one lane issues the tensor-core
        // instructions.  With the loop inside an `if (lane == 0)` the compiler has to treat every
        // address and descriptor as a per-thread value and moves each operand of each
        // tcgen05.mma into the uniform registers the instruction reads, ~100 cycles of a lone
        // thread's issue time per instruction, more than a 128x128x16 product takes (64 cycles);
        // warp-uniform control flow keeps that arithmetic on the uniform datapath.
        {
            const uint32_t idesc = p.fmt == PF_F16 ? make_idesc_f16_f32(kCBM, BN) : make_idesc_bf16_f32(kCBM, BN);
            const uint32_t idesc64 = p.fmt == PF_F16 ? make_idesc_f16_f32(kCBM, 64) : make_idesc_bf16_f32(kCBM, 64);
            constexpr int kWide = 2 * BN <= 256 ? 2 * BN : BN;  // (256-column tiles never take the packed path)
            const uint32_t idesc_wide = make_idesc_bf16_f32(kCBM, kWide);
            const uint64_t eye = make_smem_desc_sw128(smem_base + ident_off);
            const bool issuer = lane == 0;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t seg = 0;
            int kb = first_k;
            int it = first_iter;
            int num_kb = tile_kb_count(blockIdx.x + it * gridDim.x) + p.res_kb;
            bool seg_open = false;
            TCK(t_mma0);
#ifdef GPX_CGEMM_TIMING
            long long mma_wait_full = 0, mma_wait_tmem = 0, mma_kb = 0;
#endif
            for (;;) {
                TCK(t_f0);
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_flag, kCWaitLimitNs))) {
                    if (issuer) fail(201);
                    break;
                }
#ifdef GPX_CGEMM_TIMING
                mma_wait_full += clock64() - t_f0;
                ++mma_kb;
#endif
                tc_fence_after_sync();
                const int msg = __shfl_sync(0xffffffffu, ctl->stage_msg[stage], 0);
                const int buf = (int)(seg % nbuf);
                const uint32_t acc0 = tmem_base + buf * buf_cols;
                if (!seg_open) {
                    TCK(t_e0);
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&ctl->tmem_empty[buf]), (seg / nbuf) & 1, abort_flag,
                                                           kCWaitLimitNs))) {
                        if (issuer) fail(202);
                        break;
                    }
#ifdef GPX_CGEMM_TIMING
                    mma_wait_tmem += clock64() - t_e0;
#endif
                    tc_fence_after_sync();
                    seg_open = true;
                }
                if (msg != CMSG_DATA && msg < CMSG_RES) {
                    if (issuer) {
                        ctl->epi_kind[buf] = msg == CMSG_STOP ? CEPI_PARTIAL : CEPI_EXIT;
                        ctl->epi_k_done[buf] = kb;
                        mma_commit(smem_u32(&ctl->tmem_full[buf]));
                        mbar_arrive(smem_u32(&ctl->tmem_full[buf]));
                    }
                    __syncwarp();
                    break;
                }
                const uint32_t base = smem_base + stage * stage_bytes;
                const uint64_t a_hi = make_smem_desc_sw128(base);
                const uint64_t a_lo = make_smem_desc_sw128(base + Cfg::kABytes);
                const uint64_t w_hi = make_smem_desc_sw128(base + w_off);
                const uint64_t w_lo = make_smem_desc_sw128(base + 2 * Cfg::kABytes + Cfg::kWBytes);
                // fp32 product from three bf16 products.  The tensor core truncates when it adds
                // into the fp32 accumulator, a bias that grows with the length of the accumulation
                // chain, so the chain is split over several accumulators that the epilogue adds with
                // round-to-nearest.  The order is fixed, so a resumed tile replays exactly the
                // instruction sequence of an uninterrupted one.
                const uint32_t first = kb > 0 ? 1u : 0u;
                if (issuer) {
                    if (msg >= CMSG_RES) {
                        // residual x identity on 64 accumulator columns: the hi plane into a hi*hi
                        // accumulator, the lo plane into a cross-term accumulator (exact products,
                        // added like any other)
                        const uint32_t col = (uint32_t)(msg - CMSG_RES) * 64;
#pragma unroll
                        for (int k = 0; k < kCBK / kCUmmaK; ++k) {
                            if (dual && two_plane) {
                                mma_f16_ss(acc0 + col, a_hi + 2 * k, eye + 2 * k, idesc64, 1u);
                                mma_f16_ss(acc0 + BN + col, a_lo + 2 * k, eye + 2 * k, idesc64, 1u);
                            } else {
                                mma_f16_ss(acc0 + (k & 1) * BN + col, a_hi + 2 * k, eye + 2 * k, idesc64, 1u);
                                if (two_plane) mma_f16_ss(acc0 + 3 * BN + col, a_lo + 2 * k, eye + 2 * k, idesc64, 1u);
                            }
                        }
                    } else if (dual && two_plane && p.packed) {
                        // hi*hi in one accumulator, both cross terms in the other.  The W_lo tile
                        // follows the W_hi tile in the stage and the two accumulators are adjacent
                        // columns, so A_hi x [W_hi; W_lo] is ONE instruction of width 2*BN: the
                        // kernel is bound by shared-memory bandwidth (operand reads plus the TMA
                        // fill), and this reads the A_hi tile once instead of twice.  Every
                        // accumulator element still receives the same additions in the same order.
#pragma unroll
                        for (int k = 0; k < kCBK / kCUmmaK; ++k) {
                            mma_f16_ss(acc0, a_hi + 2 * k, w_hi + 2 * k, idesc_wide, (first || k > 0) ? 1u : 0u);
                            mma_f16_ss(acc0 + BN, a_lo + 2 * k, w_hi + 2 * k, idesc, 1u);
                        }
                    } else if (dual && two_plane) {
#pragma unroll
                        for (int k = 0; k < kCBK / kCUmmaK; ++k) {
                            mma_f16_ss(acc0, a_hi + 2 * k, w_hi + 2 * k, idesc, (first || k > 0) ? 1u : 0u);
                            mma_f16_ss(acc0 + BN, a_hi + 2 * k, w_lo + 2 * k, idesc, (first || k > 0) ? 1u : 0u);
                            mma_f16_ss(acc0 + BN, a_lo + 2 * k, w_hi + 2 * k, idesc, 1u);
                        }
                    } else {
                        // hi*hi terms alternate between two accumulators (even / odd K steps); the
                        // small hi*lo and lo*hi terms get one each
#pragma unroll
                        for (int k = 0; k < kCBK / kCUmmaK; ++k) {
                            mma_f16_ss(acc0 + (k & 1) * BN, a_hi + 2 * k, w_hi + 2 * k, idesc, (first || k > 1) ? 1u : 0u);
                            if (two_plane) {
                                mma_f16_ss(acc0 + 2 * BN, a_hi + 2 * k, w_lo + 2 * k, idesc, (first || k > 0) ? 1u : 0u);
                                mma_f16_ss(acc0 + 3 * BN, a_lo + 2 * k, w_hi + 2 * k, idesc, (first || k > 0) ? 1u : 0u);
                            }
                        }
                    }
                    mma_commit(smem_u32(&ctl->empty[stage]));
                }
                __syncwarp();
                if (++stage == nst) {
                    stage = 0;
                    phase ^= 1;
                }
                if (++kb == num_kb) {
                    if (issuer) {
                        ctl->epi_kind[buf] = CEPI_COMPLETE;
                        ctl->epi_k_done[buf] = num_kb;
                        mma_commit(smem_u32(&ctl->tmem_full[buf]));
                        mbar_arrive(smem_u32(&ctl->tmem_full[buf]));
                    }
                    __syncwarp();
                    ++seg;
                    ++it;
                    num_kb = tile_kb_count(blockIdx.x + it * gridDim.x) + p.res_kb;
                    kb = 0;
                    seg_open = false;
                }
            }
#ifdef GPX_CGEMM_TIMING
            if (issuer) {
                TADD(2, mma_wait_full);
                TADD(3, mma_wait_tmem);
                TADD(4, clock64() - t_mma0);
                TADD(12, mma_kb);
            }
#endif
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp & 3;
        const int part = (warp - 2) >> 2;                 // which share of the columns
        const int c_lo = part * (BN / kCEpiParts), c_hi = c_lo + BN / kCEpiParts;
        // this warp's share of the columns of one accumulator buffer, for spill and restore
        const int s_lo = part * (buf_cols / kCEpiParts), s_hi = s_lo + buf_cols / kCEpiParts;
        const int row = quarter * 32 + lane;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const bool leader = threadIdx.x == 64;
        uint32_t v[32];
        if (first_k > 0) {
            for (int c = s_lo; c < s_hi; c += 32) {
                // Spill layout: private to this kernel, so it is chosen for the stores: the j-th
                // 16-byte piece of a 32-column chunk of all 128 rows is contiguous, one warp store
                // writes 512 consecutive bytes (row-major rows 2 KB apart cost a line per thread).
                const uint4 *src = reinterpret_cast<const uint4 *>(spill) + (size_t)(c / 32) * 8 * kCBM + row;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint4 q = src[j * kCBM];
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
        asm volatile("bar.sync 1, %0;" ::"n"(kCEpiThreads) : "memory");
        if (leader)
            for (int b = 0; b < nbuf; ++b) mbar_arrive(smem_u32(&ctl->tmem_empty[b]));

        int it = first_iter;
        int seg_k0 = first_k;
        int tiles_done = 0;
        const int img = p.in_hs * p.in_ws;
        float bias_next = 0.f;  // this thread's bias element of the next tile to drain
        if (p.bias && !p.partial) {
            const int t = (int)threadIdx.x - 64;
            const int first_tile = blockIdx.x + first_iter * gridDim.x;
            if (t < BN && first_tile < total_tiles)
                bias_next = __ldg(p.bias + ((first_tile / p.k_splits) % p.tiles_n) * BN + t);
        }
        TCK(t_epi0);
#ifdef GPX_CGEMM_TIMING
        long long e_wait = 0, e_tmem = 0, e_math = 0, e_store = 0, e_bar = 0;
#endif
        for (uint32_t seg = 0;; ++seg) {
            const int buf = (int)(seg % nbuf);
            const uint32_t t_acc = t_lane + buf * buf_cols;
            TCK(t_wait0);
            // The bias of the tile this buffer holds goes to shared memory before the drain loop
            // (read from global memory inside it, its latency - an L2 round trip under load - was
            // paid once per 16-column piece).  The value stored now was requested one tile ago
            // and the request for the tile after this one is issued here, so the round trip
            // overlaps the drain of this tile instead of delaying its start.
            if (p.bias && !p.partial) {
                const int t = (int)threadIdx.x - 64;
                if (t < BN) {
                    ctl->bias_s[buf][t] = bias_next;
                    const int after = blockIdx.x + (it + 1) * gridDim.x;
                    if (after < total_tiles) bias_next = __ldg(p.bias + ((after / p.k_splits) % p.tiles_n) * BN + t);
                }
            }
            if (leader) {
                bool ok = mbar_wait(smem_u32(&ctl->tmem_full[buf]), (seg / nbuf) & 1, abort_flag, kCWaitLimitNs);
                if (!ok) fail(301);
                ctl->epi_go = ok ? 1 : 0;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kCEpiThreads) : "memory");
#ifdef GPX_CGEMM_TIMING
            e_wait += clock64() - t_wait0;
#endif
            if (!ctl->epi_go) break;
            tc_fence_after_sync();
            const int kind = ctl->epi_kind[buf];
            const int k_done = ctl->epi_k_done[buf];
            if (kind == CEPI_EXIT) {
                if (leader && resumable) {
                    slot->next_iter = it;
                    slot->k_done = 0;
                    slot->grid = gridDim.x;
                }
                break;
            }
            if (kind == CEPI_COMPLETE) {
                const int tile = blockIdx.x + it * gridDim.x;
                int otile = tile, split = 0;
                if (p.k_splits > 1) {
                    otile = fast_div(tile, p.k_splits, p.inv_k_splits);
                    split = tile - otile * p.k_splits;
                }
                const int m_blk = p.tiles_n > 1 ? fast_div(otile, p.tiles_n, p.inv_tiles_n) : otile;
                const int n_blk = otile - m_blk * p.tiles_n;
                // Which output pixel, if any, does this GEMM row stand for?
                const int vrow = m_blk * kCBM + row;
                bool valid = vrow < p.m_rows;
                size_t out_off = 0, res_off = 0;
                if (p.identity_rows) {
                    // plain rows in, plain rows out (and a plain residual): row m of the GEMM is
                    // row m of the output, no pixel arithmetic is needed
                    if (valid) {
                        out_off = (size_t)vrow * p.out.C + (size_t)n_blk * BN;
                        if (p.res_hi) res_off = (size_t)vrow * p.res.C + (size_t)n_blk * BN;
                    }
                } else {
                    int n_img = 0, h = 0, w = 0;
                    if (valid) {
                        n_img = fast_div(vrow, img, p.inv_img);
                        int r = vrow - n_img * img;
                        int hs = fast_div(r, p.in_ws, p.inv_in_ws);
                        int ws = r - hs * p.in_ws;
                        h = hs - p.in_off;
                        w = ws - p.in_off;
                        valid = h >= 0 && h < p.out.H && w >= 0 && w < p.out.W;
                    }
                    if (valid) {
                        out_off = p.out_f32 ? ((size_t)(n_img * p.out.H + h) * p.out.W + w) * p.cout_valid
                                            : (size_t)layout_row(p.out, n_img, h, w) * p.out.C + (size_t)n_blk * BN;
                        if (p.res_hi) res_off = (size_t)layout_row(p.res, n_img, h, w) * p.res.C + (size_t)n_blk * BN;
                    }
                }
                // Every lane owns one row of the tile (its TMEM lane): 16 columns of a plane are 32
                // contiguous bytes of that row, one 256-bit access, a whole sector.
                const bool planes_out = !p.partial && !p.out_f32;
                const int col_lim = p.cout_valid - n_blk * BN;
                for (int c = c_lo; c < c_hi; c += 16) {
                    float f[16];
                    uint32_t t16[16];
                    // The residual is requested first so its latency overlaps the TMEM reads.
                    const bool use_res = planes_out && p.res_hi && valid;
                    TCK(t_p0);
                    uint32_t rh[8], rl[8];
                    if (use_res) {
                        ld_global_v8(p.res_hi + res_off + c, rh);
                        if (two_plane) ld_global_v8(p.res_lo + res_off + c, rl);
                    }
                    {
                        uint32_t u16[16];
                        tmem_ld_32x16(t_acc + c, t16);
                        tmem_ld_32x16(t_acc + BN + c, u16);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(t16[j]) + __uint_as_float(u16[j]);
                    }
                    if (two_plane && !dual) {
                        tmem_ld_32x16(t_acc + 2 * BN + c, t16);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) f[j] += __uint_as_float(t16[j]);
                        tmem_ld_32x16(t_acc + 3 * BN + c, t16);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) f[j] += __uint_as_float(t16[j]);
                    }
#ifdef GPX_CGEMM_TIMING
                    long long t_p1 = clock64();
                    e_tmem += t_p1 - t_p0;
#endif
                    if (p.cluster_reduce) {
                        // Split K inside a cluster: the raw fp32 sum of this K range stays in this
                        // CTA's shared memory (the ring is idle: a CTA of such a launch runs one
                        // tile); rows are 16 bytes longer than BN floats so that the 32 rows of a
                        // warp spread over the banks.
                        float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(smem) + (size_t)row * (BN + 4) + c);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            dst[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                        continue;
                    }
                    if (p.partial) {
                        // Split K: the raw fp32 sum of this K range goes to the workspace; the
                        // finishing kernel adds the ranges in split order and applies the rest.
                        if (vrow < p.m_rows) {
                            float4 *dst = reinterpret_cast<float4 *>(
                                p.partial + ((size_t)split * p.partial_rows + vrow) * p.partial_ld + n_blk * BN + c);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                dst[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                        }
                        continue;
                    }
                    if (p.bias) {
                        const float4 *b4 = reinterpret_cast<const float4 *>(&ctl->bias_s[buf][c]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float4 b = b4[j];
                            f[4 * j + 0] += b.x;
                            f[4 * j + 1] += b.y;
                            f[4 * j + 2] += b.z;
                            f[4 * j + 3] += b.w;
                        }
                    }
                    if (use_res) {
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            float2 r = pf_unpack2(rh[q], p.fmt);
                            f[2 * q] += r.x;
                            f[2 * q + 1] += r.y;
                        }
                        if (two_plane) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                f[2 * q] += bf16_lo_to_f32(rl[q]);
                                f[2 * q + 1] += bf16_hi_to_f32(rl[q]);
                            }
                        }
                    }
                    apply_act_n(f, p.relu);
                    if (p.out_f32) {
                        const int col0 = n_blk * BN + c;
                        if (valid) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (col0 + j < p.cout_valid) p.out_f32[out_off + col0 + j] = f[j];
                        }
                        continue;
                    }
                    uint32_t hi[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) hi[q] = pf_pack2(f[2 * q], f[2 * q + 1], p.fmt);
                    // The output may be a channel slice: nothing is stored past cout_valid.
                    const bool store = valid && c < col_lim;
#ifdef GPX_CGEMM_TIMING
                    long long t_p2 = clock64();
                    e_math += t_p2 - t_p1;
#endif
                    if (store) st_global_v8(p.out_hi + out_off + c, hi);
                    if (two_plane) {
                        uint32_t lo[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            lo[q] = pack_bf16(f[2 * q] - bf16_lo_to_f32(hi[q]), f[2 * q + 1] - bf16_hi_to_f32(hi[q]));
                        if (store) st_global_v8(p.out_lo + out_off + c, lo);
                    }
#ifdef GPX_CGEMM_TIMING
                    e_store += clock64() - t_p2;
#endif
                }
                ++it;
                ++tiles_done;
                seg_k0 = 0;
                tc_fence_before_sync();
                TCK(t_b0);
                asm volatile("bar.sync 1, %0;" ::"n"(kCEpiThreads) : "memory");
#ifdef GPX_CGEMM_TIMING
                e_bar += clock64() - t_b0;
#endif
                if (leader) {
                    mbar_arrive(smem_u32(&ctl->tmem_empty[buf]));
                    if (blp.executed) atomicAdd(blp.executed, 1);
                }
                continue;
            }
            // CEPI_PARTIAL
            const int keep_k = p.drop_on_stop ? 0 : k_done;
            if (keep_k > seg_k0) {
                for (int c = s_lo; c < s_hi; c += 32) {
                    tmem_ld_32x32(t_acc + c, v);
                    tmem_ld_wait();
                    uint4 *dst = reinterpret_cast<uint4 *>(spill) + (size_t)(c / 32) * 8 * kCBM + row;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        dst[j * kCBM] = make_uint4(v[4 * j + 0], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
            if (leader) {
                slot->next_iter = it;
                slot->k_done = keep_k;
                slot->grid = gridDim.x;
                if (blp.stop_index) atomicCAS(blp.stop_index, -1, blp.kernel_id);
            }
            break;
        }
        if (leader && blp.trace && tiles_done) atomicAdd(blp.trace + 3, (unsigned long long)tiles_done);
#ifdef GPX_CGEMM_TIMING
        if (lane == 0) {
            TADD(5, e_wait);
            TADD(6, e_tmem);
            TADD(7, e_math);
            TADD(8, e_store);
            TADD(9, e_bar);
            TADD(10, clock64() - t_epi0);
        }
        if (leader) TADD(11, tiles_done);
#endif
    }

    tc_fence_before_sync();
    __syncthreads();
    if (p.cluster_reduce) {
        // Every CTA of the cluster has left its partial tile in shared memory (or has failed and set
        // the error word: all waits above are bounded, so every thread gets here).  CTA r finishes
        // rows [r, r+1) * 128/S of the output block: the S partial rows are read through distributed
        // shared memory and added in split order from zero, exactly as splitk_finish_kernel adds the
        // workspace rows, then bias, residual, activation and store by the same function.
        cluster_sync_all();
        if (warp >= 2) {
            const int S = p.k_splits;
            const int rank = (int)cluster_ctarank();
            const int otile = (int)blockIdx.x / S;
            const int m_blk = otile / p.tiles_n, n_blk = otile - m_blk * p.tiles_n;
            const int rows_per = kCBM / S;
            const int img = p.fin.in_hs * p.fin.in_ws;
            const uint32_t stage = smem_base;
            for (int e = (int)threadIdx.x - 64; e < rows_per * (BN / 8); e += kCEpiThreads) {
                const int lr = e / (BN / 8), c8 = e - lr * (BN / 8);
                const int trow = rank * rows_per + lr;
                const int vrow = m_blk * kCBM + trow;
                const int col0 = n_blk * BN + c8 * 8;
                if (vrow >= p.fin.m_rows || col0 >= p.fin.cout_padded) continue;
                const int n_img = vrow / img;
                const int r = vrow - n_img * img;
                const int hs = r / p.fin.in_ws;
                const int h = hs - p.fin.in_off;
                const int w = r - hs * p.fin.in_ws - p.fin.in_off;
                if (h < 0 || h >= p.fin.out.H || w < 0 || w >= p.fin.out.W) continue;
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = 0.f;
                const uint32_t local = stage + (uint32_t)(((size_t)trow * (BN + 4) + c8 * 8) * sizeof(float));
                for (int sidx = 0; sidx < S; ++sidx) {
                    const uint32_t remote = cluster_map_shared(local, (uint32_t)sidx);
                    const float4 a = ld_shared_cluster_f4(remote), b = ld_shared_cluster_f4(remote + 16);
                    f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
                    f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
                }
                splitk_apply(p.fin, n_img, h, w, col0, f);
            }
        }
        // no CTA may exit (and release its shared memory) while a peer still reads it
        cluster_sync_all();
    }
    if (warp == 0 && lane == 0 && *abort_flag) {
        for (int spin = 0; spin < 64; ++spin) __nanosleep(1000);
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
    if (threadIdx.x == 0 && blp.trace) atomicMax(blp.trace + 1, globaltimer_ns());
#ifdef GPX_CGEMM_TIMING
    if (threadIdx.x == 0) {
        TADD(13, clock64() - t_start);
        TADD(15, 1);
    }
#endif
}

#ifdef GPX_CGEMM_TIMING
// Development build only: copies the phase timers to the host and optionally clears them.
extern "C" int gpx_debug_cgemm_timing(unsigned long long *out, int reset) {
    if (cudaMemcpyFromSymbol(out, g_cgemm_timing, sizeof(unsigned long long) * 32) != cudaSuccess) return 1;
    if (reset) {
        static unsigned long long zeros[32] = {0};
        if (cudaMemcpyToSymbol(g_cgemm_timing, zeros, sizeof(zeros)) != cudaSuccess) return 1;
    }
    return 0;
}
#endif

cudaError_t cgemm_prepare(int device) {
    static bool done[64] = {false};
    if (device < 0 || device >= 64 || done[device]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(cgemm_tcgen05_kernel<128>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)CgemmCfg<128>::kSmem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(cgemm_tcgen05_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)CgemmCfg<256>::kSmem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(cgemm_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)CgemmCfg<64>::kSmem);
    if (e != cudaSuccess) return e;
    done[device] = true;
    return cudaSuccess;
}

template <int BN>
static cudaError_t cgemm_launch_cluster(const CgemmParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)kCgemmThreads);
    cfg.dynamicSmemBytes = CgemmCfg<BN>::kSmem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    at[1].id = cudaLaunchAttributeClusterDimension;
    at[1].val.clusterDim.x = (unsigned)p.k_splits;
    at[1].val.clusterDim.y = 1;
    at[1].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, cgemm_tcgen05_kernel<BN>, p, blp);
}

// CTAs of clusters of `cluster` CTAs of this kernel that the device keeps resident at once.
int cgemm_max_cluster(int bn, int cluster) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)cluster);
    cfg.blockDim = dim3((unsigned)kCgemmThreads);
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)cluster;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int clusters = 0;
    cudaError_t err;
    if (bn == 128) {
        cfg.dynamicSmemBytes = CgemmCfg<128>::kSmem;
        err = cudaOccupancyMaxActiveClusters(&clusters, cgemm_tcgen05_kernel<128>, &cfg);
    } else {
        cfg.dynamicSmemBytes = CgemmCfg<64>::kSmem;
        err = cudaOccupancyMaxActiveClusters(&clusters, cgemm_tcgen05_kernel<64>, &cfg);
    }
    if (err != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return clusters * cluster;
}

cudaError_t cgemm_launch(const CgemmParams &p, int bn, int grid, const BlpArgs &blp, cudaStream_t s) {
    if (p.cluster_reduce) {
        // (256-column tiles are never split)
        if (bn == 128) return cgemm_launch_cluster<128>(p, grid, blp, s);
        return cgemm_launch_cluster<64>(p, grid, blp, s);
    }
    if (bn == 256)
        launch_layer(cgemm_tcgen05_kernel<256>, grid, kCgemmThreads, CgemmCfg<256>::kSmem, s, p, blp);
    else if (bn == 128)
        launch_layer(cgemm_tcgen05_kernel<128>, grid, kCgemmThreads, CgemmCfg<128>::kSmem, s, p, blp);
    else
        launch_layer(cgemm_tcgen05_kernel<64>, grid, kCgemmThreads, CgemmCfg<64>::kSmem, s, p, blp);
    return cudaGetLastError();
}

int cgemm_threads() { return kCgemmThreads; }

size_t cgemm_spill_floats_per_cta() { return (size_t)kCBM * CgemmCfg<128>::kTmemCols; }

}  // namespace gpx
