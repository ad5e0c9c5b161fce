// Persistent, warp-specialised tcgen05 GEMM core for sm_100a.
//
//   D[m, n] = sum_k A[m, k] * B[n, k]        (fp32 accumulation in tensor memory)
//
// Operands are 16-bit (bf16 or fp16) and arrive through TMA tensor maps into 128-byte-swizzled
// shared memory. Either operand may be K-major (k contiguous in global memory) or MN-major
// (m resp. n contiguous), so that X·Wᵀ, G·W and Gᵀ·X all run on this one main loop without a
// transposed copy of anything. The result never leaves the chip as a matrix: an epilogue functor
// receives every 128 x BN accumulator tile as "one thread = one row, 32 columns at a time" and
// decides what reaches global memory (softmax statistics, the logit-gradient band, dX, dW).
//
// CTA layout (192 threads):
//   warp 0      TMA producer   (one elected lane)
//   warp 1      tensor-memory allocator + tcgen05.mma issuer (one elected lane)
//   warps 2-5   epilogue; warp w owns TMEM lanes 32*(w%4) .. 32*(w%4)+31
// Pipelines: STAGES-deep smem ring (full/empty mbarriers) between producer and issuer, and two
// accumulator buffers in TMEM (tmem_full/tmem_empty) so the epilogue of tile i overlaps the main
// loop of tile i+1. Tiles are dealt to a persistent grid either round-robin (static) or, for launches of
// many waves, from a global counter (dynamic): the producer of each CTA (pair) draws the index of its next
// tile with an atomicAdd one tile ahead and hands it to the other roles through a small ring in shared
// memory. Dynamic dealing keeps the set of tiles in flight a contiguous window of the tile order, whatever
// the speed of the individual SMs; with the static deal slower CTAs fall behind by whole waves over a long
// launch, the operand panels they share with their neighbours have left L2 by the time they need them, and
// DRAM traffic grows to several times the algorithmic bytes.
//
// Around the main loop: the kernel sets itself up (barriers, tensor memory, cluster barrier) before it waits for
// its predecessor in the stream (programmatic dependent launch), so consecutive launches overlap by that much;
// the epilogue reads tensor memory two chunks deep; an epilogue that has a finish() step can have the LAST CTA to
// complete run it (a device counter that wraps to zero), which folds a small tail kernel into the launch; and
// a launch may carry a second, independent product (SecondGemm) whose tiles join the same deal.
//
// Two variants, selected by CG:
//   CG = 1  one CTA per tile: tcgen05.mma.cta_group::1, M = 128. 48 KB per stage (A 16 + B 32).
//   CG = 2  a CTA PAIR (cluster of 2 on one TPC) per 256 x BN tile: tcgen05.mma.cta_group::2 with
//           M = 256, issued by the even CTA for both. Each CTA loads its own 128 rows of A and
//           only HALF of the B tile (BN/2 rows); the tensor cores of the pair read both halves.
//           Per FLOP that is 2/3 of the shared-memory fill and L2 traffic of CG = 1, and the
//           32 KB stages leave room for a deeper ring. No TMA multicast is used: every copy lands
//           in the shared memory of the CTA that issued it. Cross-CTA signalling:
//             full[s]   lives in the leader: its producer announces the bytes of BOTH CTAs'
//                       copies there and both CTAs' copies count on it (the peer's producer only
//                       issues copies; it can do so as soon as its own empty[s] fires, which the
//                       same commit fires in both CTAs, so the phase it signals is always open);
//             empty[s], tmem_full[b]  local to each CTA; the leader's tcgen05.commit arrives on
//                       the barrier at that offset in both CTAs;
//             tmem_empty[b]  lives in the leader; the epilogue warps of both CTAs arrive on it.
#pragma once

#include "ptx.cuh"

namespace lce {

constexpr int kBM = 128;      // accumulator tile rows per CTA (= TMEM lanes)
constexpr int kBK = 64;       // k elements per pipeline stage (= one 128-byte swizzle row)
constexpr int kUmmaK = 16;    // k elements per tcgen05.mma for 16-bit operands
constexpr int kGemmThreads = 192;

// error codes written to the device status word
constexpr int kDevErrProducerTimeout = 101;
constexpr int kDevErrMmaTimeout = 102;
constexpr int kDevErrEpilogueTimeout = 103;
constexpr int kDevErrSchedTimeout = 104;
constexpr int kSchedSlots = 4;  // depth of the tile-index ring of the dynamic scheduler

struct TileCtx {
    int m_tile;       // 128-row tile index
    int n_tile;       // tile column index
    int n_tiles;      // tile columns in the problem
    int row_in_tile;  // 0..127, the row this thread owns
    int bn;           // tile width in columns
    int k_slice;      // which slice of the contraction this tile holds (0 unless K is split)
    float* stage;     // this warp's 32 x 33 floats of shared memory for re-shaping a chunk, or nullptr
};

constexpr int kStageFloatsPerWarp = 32 * 33;

template <int BN, int STAGES, int CG>
struct GemmSmem {
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBRows = BN / CG;  // B rows (n indices) this CTA stages
    static constexpr int kBBytes = kBRows * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kEpiStageBytes = 4 * kStageFloatsPerWarp * 4;  // one re-shaping area per epilogue warp
    // 1024 bytes of slack so the ring can be aligned to the swizzle atom by hand
    static constexpr int kTotalBytes = STAGES * kStageBytes + kBarrierBytes + kEpiStageBytes + 1024;
};

// Tile order. The tile grid (m_units x n_tiles) is cut into bands along one dimension; inside a band
// consecutive tile indices walk the banded dimension first. CTAs that run together therefore share
// the panels of the OTHER operand, and the band's own panels (band width x K) are what must stay
// resident in L2 while the other operand streams through once per band.
//   raster > 0:  bands of `raster` row units (m fastest inside a band)   - X.W^T passes: the band of X
//                stays in L2 while W streams; raster >= m_units is plain "rows first".
//   raster < 0:  bands of `-raster` tile columns (n fastest inside)      - dW / dX passes.
__device__ __forceinline__ void tile_coords(int tile, int m_units, int n_tiles, int raster,
                                            int& m_unit, int& n_tile) {
    if (raster > 0) {
        const int band_tiles = raster * n_tiles;
        const int band = tile / band_tiles;
        const int r = tile - band * band_tiles;
        const int w = min(raster, m_units - band * raster);
        n_tile = r / w;
        m_unit = band * raster + (r - n_tile * w);
    } else {
        const int wb = -raster;
        const int band_tiles = wb * m_units;
        const int band = tile / band_tiles;
        const int r = tile - band * band_tiles;
        const int w = min(wb, n_tiles - band * wb);
        m_unit = r / w;
        n_tile = band * wb + (r - m_unit * w);
    }
}

// m_tiles counts 128-row tiles. With CG = 2 the scheduler deals out pairs of them: unit u covers
// m tiles 2u and 2u+1 (the second may lie past the end of the matrix: its loads return zeros
// and the epilogues skip its rows).
// k_splits > 1 splits the contraction: work item w = (tile unit w % units, slice w / units) covers
// k blocks [slice * per, (slice+1) * per) and hands the epilogue a partial sum tagged with its slice
// (the epilogue stores slices side by side; a later pass adds them in slice order). The host
// guarantees that every slice is non-empty.
// An optional SECOND product computed by the same launch (same tile shape, B layout, element type and epilogue
// kind; its own operands, sizes, A layout and epilogue parameters). Its work items follow the first product's in
// the round-robin deal, so two small independent products - the backward's dX and dW for a handful of tokens -
// share one launch instead of running one after the other. Static deal only.
struct NoSecondGemm {
    static constexpr bool kPresent = false;
    static constexpr bool kAMn = false;
};
template <class Epi, bool A_MN2>
struct SecondGemm {
    static constexpr bool kPresent = true;
    static constexpr bool kAMn = A_MN2;
    CUtensorMap tmA, tmB;
    int m_tiles, n_tiles, k_blocks, k_splits, raster;
    typename Epi::Params ep;
};

template <int BN, int STAGES, int CG, bool A_MN, bool B_MN, bool IS_BF16, class Epi, class Second = NoSecondGemm>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               int m_tiles, int n_tiles, int k_blocks, int k_splits, int raster, int l2_hints,
               const typename Epi::Params ep, int* __restrict__ status, int* __restrict__ sched_counter,
               unsigned* __restrict__ done_counter, const __grid_constant__ Second second = Second{}) {
    using S = GemmSmem<BN, STAGES, CG>;
    static_assert(CG == 1 || CG == 2, "cta group");
    static_assert(BN % (64 * CG) == 0 && BN >= 64 && BN <= 256, "tile width");
    static_assert(2 * BN <= 512, "two accumulator buffers must fit in tensor memory");
    constexpr uint32_t kTmemCols = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);
    constexpr uint32_t kIdesc = ptx::make_idesc_f16(kBM * CG, BN, IS_BF16, A_MN, B_MN);
    constexpr uint32_t kIdesc2 = ptx::make_idesc_f16(kBM * CG, BN, IS_BF16, Second::kAMn, B_MN);
    constexpr bool kPair = CG == 2;
    constexpr bool kDual = Second::kPresent;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + STAGES * S::kStageBytes;
    // barrier block: full[STAGES] | empty[STAGES] | tmem_full[2] | tmem_empty[2] | drain | tmem ptr | abort
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
    uint8_t* gen_bar_base = smem_raw + (bar_base - ptx::smem_u32(smem_raw));
    volatile uint32_t* tmem_ptr_smem =
        reinterpret_cast<volatile uint32_t*>(gen_bar_base + 8 * (2 * STAGES + 5));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_bar_base + 8 * (2 * STAGES + 5) + 4);
    // dynamic scheduler: sched_full[kSchedSlots] | sched_empty[kSchedSlots] | tile index per slot
    auto sfull_bar = [&](int q) { return bar_base + 8u * (2 * STAGES + 6 + q); };
    auto sempty_bar = [&](int q) { return bar_base + 8u * (2 * STAGES + 6 + kSchedSlots + q); };
    const uint32_t sched_tiles = bar_base + 8u * (2 * STAGES + 6 + 2 * kSchedSlots);
    volatile int* sched_tile_gen = reinterpret_cast<volatile int*>(gen_bar_base + 8 * (2 * STAGES + 6 + 2 * kSchedSlots));
    static_assert(8 * (2 * STAGES + 6 + 2 * kSchedSlots) + 4 * kSchedSlots <= S::kBarrierBytes, "barrier block too small");
    const bool dyn = sched_counter != nullptr;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;  // 0 = leader of the pair
    const int unit0 = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int unit_step = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int m_units = kPair ? (m_tiles + 1) / 2 : m_tiles;
    const int total_units = m_units * n_tiles;
    const int work_first = total_units * k_splits;  // work items of the first product
    const int kb_per_slice = (k_blocks + k_splits - 1) / k_splits;
    int total_work = work_first;
    if constexpr (kDual)
        total_work += (kPair ? (second.m_tiles + 1) / 2 : second.m_tiles) * second.n_tiles * second.k_splits;
    // Which product a work item belongs to, and that product's tiling.
    struct Item {
        bool sec;
        int w, m_units, n_tiles, total_units, k_blocks, kb_per_slice, raster;
    };
    auto item_of = [&](int work) {
        Item it{false, work, m_units, n_tiles, total_units, k_blocks, kb_per_slice, raster};
        if constexpr (kDual) {
            if (work >= work_first) {
                it.sec = true;
                it.w = work - work_first;
                it.m_units = kPair ? (second.m_tiles + 1) / 2 : second.m_tiles;
                it.n_tiles = second.n_tiles;
                it.total_units = it.m_units * it.n_tiles;
                it.k_blocks = second.k_blocks;
                it.kb_per_slice = (second.k_blocks + second.k_splits - 1) / second.k_splits;
                it.raster = second.raster;
            }
        }
        return it;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);  // the (leader's) producer; copies count bytes on it
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), 4 * CG);  // one arrival per epilogue warp of the group
        }
        ptx::mbar_init(drain_bar, 1);
        for (int q = 0; q < kSchedSlots; ++q) {
            ptx::mbar_init(sfull_bar(q), 1);  // the leader's producer publishes
            // readers of a slot: MMA issuer, the epilogue warps of the group, the peer's producer
            ptx::mbar_init(sempty_bar(q), 1 + 4 * CG + (CG - 1));
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
    }
    if (warp == 1) {
        if constexpr (kPair) {
            ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) ptx::cluster_sync_all();  // the peer's barriers exist before anyone signals them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    // Everything above touched no global memory. From here on the kernel reads what its predecessor in the
    // stream wrote (operands, row factors, the tile counter): wait for it, and let the successor begin its own
    // set-up now (it waits the same way before it reads anything of ours).
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();

    // Reader side of the tile deal: the work item that follows the `seq`-th one this CTA handled.
    // Static deal: the next one round-robin. Dynamic deal: what the leader's producer put into ring slot
    // seq % kSchedSlots (a value >= total_work ends the loop); the slot is released on the leader's barrier.
    auto next_work = [&](int work, uint32_t seq, bool release, bool& ok) -> int {
        if (!dyn) return work + unit_step;
        const uint32_t q = seq % kSchedSlots, par = (seq / kSchedSlots) & 1u;
        if (!ptx::mbar_wait_cluster(sfull_bar(q), par, abort_flag)) {
            ok = false;
            return total_work;
        }
        const int nxt = sched_tile_gen[q];
        if (release) {
            if constexpr (kPair) ptx::mbar_arrive_cluster(ptx::map_to_cta(sempty_bar(q), 0));
            else ptx::mbar_arrive(sempty_bar(q));
        }
        return nxt;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            uint32_t issued = 0;
            bool ok = true;
            const uint32_t leader_full0 = kPair ? ptx::map_to_cta(full_bar(0), 0) : 0u;
            // l2_hints: eviction priority of operand A in bits 0-1, of operand B in bits 2-3
            const uint64_t policy_a = ptx::make_l2_policy(l2_hints & 3);
            const uint64_t policy_b = ptx::make_l2_policy((l2_hints >> 2) & 3);
            const uint32_t announce_extra = ptx::g_debug_announce_extra;  // test hook: 0 outside the wait-expiry test
            // dynamic deal (leader only): `nxt` is the work item after the current one, drawn one tile ahead
            int nxt = total_work, drawn = total_work;
            uint32_t seq = 0;
            if (dyn && cta_rank == 0) nxt = unit_step + atomicAdd(sched_counter, 1);
            for (int work = unit0; work < total_work && ok;) {
                if (dyn && cta_rank == 0) {
                    // publish the successor of this tile to the other roles (and to the peer CTA), then draw
                    // the one after it: its value is not needed before the next iteration
                    const uint32_t q = seq % kSchedSlots, par = (seq / kSchedSlots) & 1u;
                    if (!ptx::mbar_wait_cluster(sempty_bar(q), par ^ 1u, abort_flag)) {
                        atomicCAS(status, 0, kDevErrSchedTimeout);
                        ok = false;
                        break;
                    }
                    sched_tile_gen[q] = nxt;
                    if constexpr (kPair) {
                        ptx::st_shared_cluster_u32(ptx::map_to_cta(sched_tiles + 4u * q, 1), static_cast<uint32_t>(nxt));
                        ptx::mbar_arrive_cluster(ptx::map_to_cta(sfull_bar(q), 1));
                    }
                    ptx::mbar_arrive(sfull_bar(q));
                    drawn = nxt < total_work ? unit_step + atomicAdd(sched_counter, 1) : total_work;
                }
                int m_unit, n_tile;
                const Item it = item_of(work);
                tile_coords(it.w % it.total_units, it.m_units, it.n_tiles, it.raster, m_unit, n_tile);
                const int kb_begin = (it.w / it.total_units) * it.kb_per_slice;
                const int kb_end = min(it.k_blocks, kb_begin + it.kb_per_slice);
                const int m_tile = kPair ? 2 * m_unit + static_cast<int>(cta_rank) : m_unit;
                const int b_row0 = n_tile * BN + static_cast<int>(cta_rank) * S::kBRows;
                const CUtensorMap* ta = &tmA;
                const CUtensorMap* tb = &tmB;
                bool a_mn = A_MN;
                if constexpr (kDual) {
                    if (it.sec) {
                        ta = &second.tmA;
                        tb = &second.tmB;
                        a_mn = Second::kAMn;
                    }
                }
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    const uint32_t stage = issued % STAGES;
                    const uint32_t phase = (issued / STAGES) & 1u;
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sa = smem_base + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    // the barrier the MMA issuer waits on: our own, or the leader's for a pair
                    const uint32_t fb = kPair ? leader_full0 + 8u * stage : full_bar(stage);
                    auto load = [&](uint32_t dst, const CUtensorMap* tm, int x, int y) {
                        const uint64_t policy = (tm == ta) ? policy_a : policy_b;
                        if constexpr (kPair) ptx::tma_load_2d_pair_hint(dst, tm, fb, x, y, policy);
                        else ptx::tma_load_2d_hint(dst, tm, fb, x, y, policy);
                    };
                    // bytes of the whole group's copies for this stage, announced by the leader only
                    if (cta_rank == 0)
                        ptx::mbar_arrive_expect_tx(full_bar(stage), S::kStageBytes * CG + (issued == 0 ? announce_extra : 0u));
                    if (!a_mn) {  // a constant unless the launch carries a second product
                        load(sa, ta, kb * kBK, m_tile * kBM);
                    } else {
#pragma unroll
                        for (int j = 0; j < kBM / 64; ++j)
                            load(sa + j * (kBK * 128), ta, m_tile * kBM + j * 64, kb * kBK);
                    }
                    if constexpr (!B_MN) {
                        load(sb, tb, kb * kBK, b_row0);
                    } else {
#pragma unroll
                        for (int j = 0; j < S::kBRows / 64; ++j)
                            load(sb + j * (kBK * 128), tb, b_row0 + j * 64, kb * kBK);
                    }
                    ++issued;
                }
                if (!ok) break;
                if (dyn && cta_rank == 0) {
                    work = nxt;
                    nxt = drawn;
                } else {
                    work = next_work(work, seq, true, ok);
                }
                ++seq;
            }
            if (!ok || *abort_flag) {
                // Unwinding: give every copy already in flight time to land before the CTA retires.
                if (!ok) atomicCAS(status, 0, kDevErrProducerTimeout);
                if constexpr (!kPair) {
                    const uint32_t back = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
                    for (uint32_t j = 1; j <= back; ++j) {
                        const uint32_t i = issued - j;
                        const uint32_t bar = full_bar(i % STAGES);
                        const uint32_t par = (i / STAGES) & 1u;
                        for (int spin = 0; spin < (1 << 16); ++spin)
                            if (ptx::mbar_try_wait(bar, par)) break;
                    }
                } else {
                    // the completion barrier may be the peer's: wait out the copy latency instead
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (ptx::globaltimer_ns() - t0 < 200000ull) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (cta_rank == 0 && ptx::elect_one()) {
            uint32_t consumed = 0;
            uint32_t local_tile = 0;
            bool ok = true;
            for (int work = unit0; work < total_work && ok; ++local_tile) {
                const Item it = item_of(work);
                const int kb_begin = (it.w / it.total_units) * it.kb_per_slice;
                const int kb_end = min(it.k_blocks, kb_begin + it.kb_per_slice);
                const bool a_mn = it.sec ? Second::kAMn : A_MN;
                const uint32_t idesc = it.sec ? kIdesc2 : kIdesc;
                const uint32_t buf = local_tile & 1u;
                const uint32_t buf_phase = (local_tile >> 1) & 1u;
                if (!ptx::mbar_wait(tempty_bar(buf), buf_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    const uint32_t stage = consumed % STAGES;
                    const uint32_t phase = (consumed / STAGES) & 1u;
                    if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t sa = smem_base + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        // K-major: 16 elements = 32 bytes further along the swizzled row.
                        // MN-major: 16 k-rows of 128 bytes further down.
                        const uint64_t da =
                            a_mn ? ptx::make_smem_desc(sa + k * (kUmmaK * 128), kBK * 128, 1024)
                                 : ptx::make_smem_desc(sa + k * (kUmmaK * 2), 0, 1024);
                        const uint64_t db =
                            B_MN ? ptx::make_smem_desc(sb + k * (kUmmaK * 128), kBK * 128, 1024)
                                 : ptx::make_smem_desc(sb + k * (kUmmaK * 2), 0, 1024);
                        const uint32_t acc = (kb != kb_begin || k != 0) ? 1u : 0u;  // first MMA of a tile overwrites
                        if constexpr (kPair) ptx::umma_f16_pair(tmem_d, da, db, idesc, acc);
                        else ptx::umma_f16(tmem_d, da, db, idesc, acc);
                    }
                    // smem slot reusable (in both CTAs of a pair) once these MMAs retire
                    if constexpr (kPair) ptx::umma_commit_pair(empty_bar(stage), 3);
                    else ptx::umma_commit(empty_bar(stage));
                    ++consumed;
                }
                if (ok) {  // accumulator complete
                    if constexpr (kPair) ptx::umma_commit_pair(tfull_bar(buf), 3);
                    else ptx::umma_commit(tfull_bar(buf));
                    work = next_work(work, local_tile, true, ok);
                }
            }
            if (!ok || *abort_flag) {
                if (!ok) atomicCAS(status, 0, kDevErrMmaTimeout);
                // Unwinding: wait (bounded) for the MMAs already issued before TMEM is freed.
                if constexpr (kPair) ptx::umma_commit_pair(drain_bar, 1);
                else ptx::umma_commit(drain_bar);
                for (int spin = 0; spin < (1 << 16); ++spin)
                    if (ptx::mbar_try_wait(drain_bar, 0)) break;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;
        uint32_t local_tile = 0;
        bool ok = true;
        typename Epi::State st;
        for (int work = unit0; work < total_work && ok; ++local_tile) {
            int m_unit, n_tile;
            const Item it = item_of(work);
            tile_coords(it.w % it.total_units, it.m_units, it.n_tiles, it.raster, m_unit, n_tile);
            const int m_tile = kPair ? 2 * m_unit + static_cast<int>(cta_rank) : m_unit;
            const uint32_t buf = local_tile & 1u;
            const uint32_t buf_phase = (local_tile >> 1) & 1u;
            TileCtx tc{m_tile, n_tile, it.n_tiles, quarter * 32 + lane, BN, it.w / it.total_units,
                       reinterpret_cast<float*>(gen_bar_base + S::kBarrierBytes) + (warp - 2) * kStageFloatsPerWarp};
            const typename Epi::Params* epp = &ep;  // this product's epilogue parameters
            if constexpr (kDual) {
                if (it.sec) epp = &second.ep;
            }
            Epi::begin(st, *epp, tc);  // global loads for this row overlap the wait below
            if (!ptx::mbar_wait(tfull_bar(buf), buf_phase, abort_flag)) {
                ok = false;
                break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            // two chunks in flight: the tensor-memory read of the next chunk runs under the work on this one
            static_assert((BN / 32) % 2 == 0, "chunks are taken in pairs");
            float va[32], vb[32];
            ptx::tmem_ld_32x32(taddr, va);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c += 2) {
                ptx::tmem_ld_wait();
                ptx::tmem_ld_32x32(taddr + (c + 1) * 32, vb);
                Epi::chunk(st, *epp, tc, c * 32, va);
                ptx::tmem_ld_wait();
                if (c + 2 < BN / 32) ptx::tmem_ld_32x32(taddr + (c + 2) * 32, va);
                Epi::chunk(st, *epp, tc, (c + 1) * 32, vb);
            }
            // all TMEM reads of this buffer are done: hand it back to the MMA issuer
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (kPair) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(buf), 0));
                else ptx::mbar_arrive(tempty_bar(buf));
            }
            Epi::end(st, *epp, tc);
            // every lane reads the next work item; one lane releases the ring slot for the warp
            const int following = next_work(work, local_tile, false, ok);
            if (dyn && ok) {
                __syncwarp();
                if (lane == 0) {
                    const uint32_t q = local_tile % kSchedSlots;
                    if constexpr (kPair) ptx::mbar_arrive_cluster(ptx::map_to_cta(sempty_bar(q), 0));
                    else ptx::mbar_arrive(sempty_bar(q));
                }
            }
            work = following;
        }
        if (!ok && lane == 0) atomicCAS(status, 0, kDevErrEpilogueTimeout);
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) ptx::cluster_sync_all();  // neither CTA leaves while its peer may still touch it
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        if constexpr (kPair) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
        else ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
    // Fused tail (epilogues that have one, launches that were given a completion counter): every CTA counts
    // itself out once its outputs are visible device-wide; the one that counts last runs Epi::finish(). The
    // counter wraps to zero with the last arrival, so it needs no reset between launches.
    if constexpr (Epi::kHasFinish) {
        if (done_counter != nullptr) {
            __shared__ int counted_last;
            __threadfence();  // this thread's epilogue stores, before the CTA is counted out
            __syncthreads();
            if (threadIdx.x == 0) counted_last = atomicInc(done_counter, gridDim.x - 1) == gridDim.x - 1;
            __syncthreads();
            if (counted_last) {
                __threadfence();
                Epi::finish(ep);
            }
        }
    }
}

}  // namespace lce
