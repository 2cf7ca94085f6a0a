// Multi-head self-attention on the tcgen05 tensor cores for the single-plane (bf16 / fp16)
// models: softmax(Q K^T / sqrt(d)) V with head dimension 64, no mask, sequences up to 512.
//
// Stands in for the batch_matmul + softmax + batch_matmul kernels TVM generates for the
// reference's BERT workload (scripts/compile/compile-bert.py:33-91; replayed by
// src/executor.cpp:157-162).  One tile = (batch item, head, block of 128 queries), claimed through
// the block-level preemption loop (scripts/compile/convert_to_blp.py:39-70).  Per block of 128
// keys: S = Q K^T as one 128x128x64 product into tensor memory; every thread owns one query row
// (its TMEM lane), keeps the running maximum and normaliser of an online softmax and writes the
// probabilities as a 16-bit A operand into shared memory (128-byte swizzled, as TMA would); then
// P V as a 128x64x128 product whose B operand is the transposed value matrix (keys contiguous)
// that transpose_v_kernel prepares; the per-block result is folded into fp32 registers.
// Thread 0 issues TMA and MMA; every wait is bounded and its outcome is shared through a block
// barrier, so all threads leave together when one gives up.
//
// A tile of 128 queries x 512 keys takes ~27 us, above the 20 us drain target, so the preempt word
// is also polled once per block of 128 keys.  A CTA that sees it raised gives the tile up: nothing
// has been written yet, the tile number goes into the CTA's slot, and the relaunched CTA computes
// that tile from its first key block before it claims new ones (the reset-and-restart treatment of
// REEF, src/reef-client/reef_scheduler.cpp:316-357, at tile granularity: at most one tile of work
// per CTA is repeated, and the result is the same bits either way).
#include "layers.cuh"
#include "sm100.cuh"

namespace gpx {

using namespace sm100;

constexpr int kFaThreads = 128;
constexpr int kFaQ = 128, kFaKeys = 128, kFaD = 64;
constexpr uint32_t kFaTileBytes = 128 * 64 * 2;  // one 128-row x 64-column 16-bit tile: 16 KiB
constexpr uint32_t kFaSmem = 5 * kFaTileBytes + 1024 + 256;  // Q, K, Vt, P (two tiles), slack, control
constexpr uint32_t kFaTmemCols = 256;                        // S: 128 columns, P V: 64 columns
constexpr unsigned long long kFaWaitLimitNs = 2000000000ull;

struct FaControl {
    unsigned long long bar_q, bar_k, bar_v, bar_mma;
    uint32_t tmem_base;
    int tile;
    int abort_flag;
    int stop;  // the word was seen raised: leave at this key-block boundary
};

// 2^x, the hardware approximation (relative error ~2^-22; -inf gives 0).
__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void fa_st_v8(void *ptr, const uint32_t *r) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__global__ void __launch_bounds__(kFaThreads)
attention_tc_kernel(const __grid_constant__ AttnParams p, BlpArgs blp) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char *smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    const uint32_t sQ = smem_u32(smem), sK = sQ + kFaTileBytes, sV = sQ + 2 * kFaTileBytes,
                   sP = sQ + 3 * kFaTileBytes;
    unsigned char *pP = smem + 3 * kFaTileBytes;
    FaControl *ctl = reinterpret_cast<FaControl *>(smem + 5 * kFaTileBytes);
    volatile int *abort_flag = &ctl->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5;

    if (tid == 0) {
        mbar_init(smem_u32(&ctl->bar_q), 1);
        mbar_init(smem_u32(&ctl->bar_k), 1);
        mbar_init(smem_u32(&ctl->bar_v), 1);
        mbar_init(smem_u32(&ctl->bar_mma), 1);
        ctl->abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem_base), kFaTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    pdl_wait();  // the prologue above overlapped the predecessor's tail
    pdl_launch_dependents();
    if (tid == 0) trace_begin(blp);
    const uint32_t tmem = ctl->tmem_base;
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    const uint32_t idesc_s = p.fmt == PF_F16 ? make_idesc_f16_f32(128, 128) : make_idesc_bf16_f32(128, 128);
    const uint32_t idesc_o = p.fmt == PF_F16 ? make_idesc_f16_f32(128, 64) : make_idesc_bf16_f32(128, 64);
    auto fail = [&](int code) {
        ctl->abort_flag = 1;
        if (p.error && atomicCAS(p.error, 0, code) == 0) p.error[1] = blp.kernel_id * 1000 + (int)blockIdx.x;
    };
    // Thread 0 waits (bounded); the block barrier that follows publishes the outcome.
    auto leader_wait = [&](unsigned long long *bar, uint32_t phase, int code) {
        if (tid == 0 && !*abort_flag && !mbar_wait(smem_u32(bar), phase, abort_flag, kFaWaitLimitNs)) fail(code);
    };

    const int qblocks = (p.S + kFaQ - 1) / kFaQ;
    const int nkb = (p.S + kFaKeys - 1) / kFaKeys;
    const float scale_log2 = p.scale * 1.4426950408889634f;  // scores are exponentiated base 2
    uint32_t ph_q = 0, ph_k = 0, ph_v = 0, ph_m = 0;
    int iter = 0;
    int tiles_done = 0;
    bool dead = false;
    const bool resumable = blp.preempted != nullptr && p.slots != nullptr;
    CgemmSlot *slot = resumable ? p.slots + blockIdx.x : nullptr;
    // The tile this CTA gave up in the previous launch, if any (thread 0 only).
    int pending = (resumable && tid == 0) ? slot->next_iter - 1 : -1;
    for (; !dead; ++iter) {
        if (tid == 0) {
            int t;
            if (pending >= 0) {
                // An interrupted tile comes first; a kernel relaunched while the word is still up
                // keeps it for the next launch and reports itself as the stop point.
                if (load_word(blp.preempted) != 0) {
                    atomicCAS(blp.stop_index, -1, blp.kernel_id);
                    if (blp.trace) atomicMin(blp.trace + 2, globaltimer_ns());
                    t = -1;
                } else {
                    t = pending;
                    pending = -1;
                    slot->next_iter = 0;
                }
            } else {
                t = blp_claim(blp, iter);
            }
            ctl->tile = t;
            ctl->stop = 0;
        }
        __syncthreads();
        const int tile = ctl->tile;
        if (tile < 0) break;
        const int qb = tile % qblocks;
        const int head = (tile / qblocks) % p.heads;
        const int b = tile / (qblocks * p.heads);
        const int q0 = qb * kFaQ;
        const int col0 = head * kFaD;
        const int vt_row = (b * p.heads + head) * kFaD;
        if (tid == 0) {
            mbar_arrive_expect_tx(smem_u32(&ctl->bar_q), kFaTileBytes);
            tma_load_2d(sQ, &p.tq, smem_u32(&ctl->bar_q), col0, b * p.S + q0);
            mbar_arrive_expect_tx(smem_u32(&ctl->bar_k), kFaTileBytes);
            tma_load_2d(sK, &p.tk, smem_u32(&ctl->bar_k), col0, b * p.S);
            mbar_arrive_expect_tx(smem_u32(&ctl->bar_v), kFaTileBytes);
            tma_load_2d(sV, &p.tvt, smem_u32(&ctl->bar_v), 0, vt_row);
            tma_load_2d(sV + kFaTileBytes / 2, &p.tvt, smem_u32(&ctl->bar_v), 64, vt_row);
        }
        float m = -INFINITY, l = 0.f;
        float o[kFaD];
#pragma unroll
        for (int d = 0; d < kFaD; ++d) o[d] = 0.f;
        leader_wait(&ctl->bar_q, ph_q, 401);
        ph_q ^= 1;
        bool stopped = false;
        for (int kb = 0; kb < nkb; ++kb) {
            // The word is read at the top of every key block; its value is needed only after the
            // first product of the block, so the load's latency is hidden.
            int word_now = 0;
            if (resumable && tid == 0 && kb > 0) word_now = load_word(blp.preempted);
            // ---- S = Q K^T
            leader_wait(&ctl->bar_k, ph_k, 402);
            ph_k ^= 1;
            if (tid == 0 && !*abort_flag) {
                tc_fence_after_sync();
                const uint64_t dq = make_smem_desc_sw128(sQ), dk = make_smem_desc_sw128(sK);
#pragma unroll
                for (int k = 0; k < kFaD / 16; ++k) mma_f16_ss(tmem, dq + 2 * k, dk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                mma_commit(smem_u32(&ctl->bar_mma));
            }
            leader_wait(&ctl->bar_mma, ph_m, 403);
            ph_m ^= 1;
            if (tid == 0 && word_now != 0) ctl->stop = 1;
            __syncthreads();
            if (*abort_flag) {
                dead = true;
                break;
            }
            if (ctl->stop) {
                // Give the tile up.  The value tile of this block is the only copy still in flight.
                leader_wait(&ctl->bar_v, ph_v, 406);
                ph_v ^= 1;
                if (tid == 0) {
                    slot->next_iter = tile + 1;
                    atomicCAS(blp.stop_index, -1, blp.kernel_id);
                    if (blp.trace) atomicMin(blp.trace + 2, globaltimer_ns());
                }
                __syncthreads();
                stopped = true;
                break;
            }
            tc_fence_after_sync();
            if (tid == 0 && kb + 1 < nkb) {  // the key tile is free again: fetch the next block
                mbar_arrive_expect_tx(smem_u32(&ctl->bar_k), kFaTileBytes);
                tma_load_2d(sK, &p.tk, smem_u32(&ctl->bar_k), col0, b * p.S + (kb + 1) * kFaKeys);
            }
            // ---- online softmax of this thread's row over the 128 keys of the block
            const int key0 = kb * kFaKeys;
            uint32_t v[32];
            // Whole blocks (all 128 keys inside the sequence) skip the per-key bound test.
            const bool whole = key0 + kFaKeys <= p.S;
            float bmax = -INFINITY;  // of the raw scores: the scale is positive
#pragma unroll
            for (int c = 0; c < kFaKeys; c += 32) {
                tmem_ld_32x32(t_lane + c, v);
                tmem_ld_wait();
                if (whole) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) bmax = fmaxf(bmax, __uint_as_float(v[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (key0 + c + j < p.S) bmax = fmaxf(bmax, __uint_as_float(v[j]));
                }
            }
            const float m_new = fmaxf(m, bmax * scale_log2);
            const float alpha = fa_ex2(m - m_new);
            float lsum = 0.f;
            const int r8 = tid & 7;
            unsigned char *prow = pP + (tid >> 3) * 1024 + r8 * 128;
#pragma unroll
            for (int c = 0; c < kFaKeys; c += 32) {
                tmem_ld_32x32(t_lane + c, v);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float e0 = fa_ex2(fmaf(__uint_as_float(v[j]), scale_log2, -m_new));
                    float e1 = fa_ex2(fmaf(__uint_as_float(v[j + 1]), scale_log2, -m_new));
                    if (!whole) {
                        if (key0 + c + j >= p.S) e0 = 0.f;
                        if (key0 + c + j + 1 >= p.S) e1 = 0.f;
                    }
                    lsum += e0 + e1;
                    pk[j >> 1] = pf_pack2(e0, e1, p.fmt);
                }
                // 32 keys = four 16-byte pieces of this row, in the 128-byte swizzled layout of
                // an A tile: piece index XOR (row mod 8); keys 64..127 form the second tile.
                unsigned char *tile_row = prow + (c >> 6) * kFaTileBytes;
                const int piece0 = (c & 63) >> 3;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<uint4 *>(tile_row + (((piece0 + q) ^ r8) << 4)) =
                        make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            }
            l = l * alpha + lsum;
            m = m_new;
            fence_proxy_async();  // the probabilities were written by ordinary stores, the MMA reads them
            tc_fence_before_sync();
            leader_wait(&ctl->bar_v, ph_v, 404);
            ph_v ^= 1;
            __syncthreads();
            if (*abort_flag) {
                dead = true;
                break;
            }
            // ---- P V
            if (tid == 0) {
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < kFaKeys / 16; ++kk) {
                    const uint64_t dp = make_smem_desc_sw128(sP + (kk >> 2) * kFaTileBytes) + 2 * (kk & 3);
                    const uint64_t dv = make_smem_desc_sw128(sV + (kk >> 2) * (kFaTileBytes / 2)) + 2 * (kk & 3);
                    mma_f16_ss(tmem + 128, dp, dv, idesc_o, kk > 0 ? 1u : 0u);
                }
                mma_commit(smem_u32(&ctl->bar_mma));
            }
            leader_wait(&ctl->bar_mma, ph_m, 405);
            ph_m ^= 1;
            __syncthreads();
            if (*abort_flag) {
                dead = true;
                break;
            }
            tc_fence_after_sync();
            if (tid == 0 && kb + 1 < nkb) {  // value tile free: fetch the next block
                mbar_arrive_expect_tx(smem_u32(&ctl->bar_v), kFaTileBytes);
                tma_load_2d(sV, &p.tvt, smem_u32(&ctl->bar_v), (kb + 1) * kFaKeys, vt_row);
                tma_load_2d(sV + kFaTileBytes / 2, &p.tvt, smem_u32(&ctl->bar_v), (kb + 1) * kFaKeys + 64, vt_row);
            }
#pragma unroll
            for (int c = 0; c < kFaD; c += 32) {
                tmem_ld_32x32(t_lane + 128 + c, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) o[c + j] = fmaf(o[c + j], alpha, __uint_as_float(v[j]));
            }
            tc_fence_before_sync();  // orders these TMEM reads before the next block's products
        }
        if (dead || stopped) break;
        ++tiles_done;
        if (q0 + tid < p.S) {
            const float inv = 1.0f / l;
            uint32_t w[kFaD / 2];
#pragma unroll
            for (int d = 0; d < kFaD; d += 2) w[d >> 1] = pf_pack2(o[d] * inv, o[d + 1] * inv, p.fmt);
            bf16_bits *dst = p.out_hi + ((size_t)b * p.S + q0 + tid) * p.ld + col0;
#pragma unroll
            for (int q = 0; q < 4; ++q) fa_st_v8(dst + 16 * q, w + 8 * q);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kFaTmemCols);
    }
    if (tid == 0) trace_end(blp, tiles_done);
}

// Vt[(b*heads + h)*64 + d][key] = V[b*S + key][h*64 + d]: the value matrix with keys contiguous, the
// K-major B operand of the second product.  One tile = 64 keys of one (batch item, head).
__global__ void __launch_bounds__(256)
transpose_v_kernel(const __grid_constant__ AttnParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    __shared__ bf16_bits t[64][64 + 2];
    if (threadIdx.x == 0) trace_begin(blp);
    const int kblocks = (p.S + 63) / 64;
    int iter = 0;
    for (;; ++iter) {
        if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
        __syncthreads();
        const int tile = s_tile;
        if (tile < 0) break;
        const int kblk = tile % kblocks, bh = tile / kblocks;
        const int b = bh / p.heads, h = bh % p.heads;
        for (int e = threadIdx.x; e < 64 * 8; e += 256) {
            const int key = e >> 3, piece = e & 7;
            uint4 q = make_uint4(0u, 0u, 0u, 0u);
            if (kblk * 64 + key < p.S)
                q = *reinterpret_cast<const uint4 *>(p.v_hi + ((size_t)b * p.S + kblk * 64 + key) * p.ld + h * 64 + piece * 8);
            const bf16_bits *src = reinterpret_cast<const bf16_bits *>(&q);
#pragma unroll
            for (int j = 0; j < 8; ++j) t[key][piece * 8 + j] = src[j];
        }
        __syncthreads();
        for (int e = threadIdx.x; e < 64 * 8; e += 256) {
            const int d = e >> 3, piece = e & 7;
            if (kblk * 64 + piece * 8 < p.S) {  // S is a multiple of 8: whole pieces are in or out
                bf16_bits w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = t[piece * 8 + j][d];
                *reinterpret_cast<uint4 *>(p.vt + ((size_t)bh * 64 + d) * p.S + kblk * 64 + piece * 8) =
                    *reinterpret_cast<const uint4 *>(w);
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

cudaError_t attention_tc_prepare() {
    return cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFaSmem);
}

cudaError_t attention_tc_launch(const AttnParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(attention_tc_kernel, grid, kFaThreads, kFaSmem, s, p, blp);
    return cudaGetLastError();
}

cudaError_t transpose_v_launch(const AttnParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(transpose_v_kernel, grid, 256, 0, s, p, blp);
    return cudaGetLastError();
}

}  // namespace gpx
