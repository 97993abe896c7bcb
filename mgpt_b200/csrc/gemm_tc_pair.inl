// Token-major products on CTA PAIRS (included by gemm_tc.cu inside its unnamed namespace).
//
// A single CTA's 128x256 tile needs 48 KiB of operands per 64 channels, and the kernels built on it sit at what one
// SM can pull out of L2.  Here a cluster of two CTAs on neighbouring SMs computes 256x256: two 128-row tiles of ONE
// expert against the same 256 weight rows.  Each CTA loads its own 128 token rows and HALF of the weight rows (no
// multicast: plain TMA loads, each into the loading CTA's own shared memory), the leader CTA issues
// tcgen05.mma.cta_group::2 (M = 256), which reads A and its B half from each CTA's shared memory and accumulates each
// CTA's 128 rows into that CTA's TMEM.  Operand bytes per flop fall by a third; the epilogue is the single-CTA one,
// each CTA on its own rows.
//
// The plan pairs row tiles within an expert (pairs[2i], pairs[2i+1]; the second is -1 for an expert's odd last
// tile: the peer CTA then feeds the first tile's rows again and stores nothing).
//
// Synchronisation between the two CTAs, all through mbarriers with bounded waits:
//   full[s]      leader only.  The leader's producer arms it with the bytes of BOTH CTAs' loads; the peer's loads
//                count on it too (cp.async.bulk.tensor ... .cta_group::2 with the leader's barrier address).
//   empty[s]     in each CTA, released by a tcgen05.commit of the leader's MMA thread addressed to that CTA.
//   acc_full[b]  in each CTA, same mechanism.      acc_empty[b]  leader only, one arrival per epilogue warp of both CTAs.
//   work queue   the leader's producer takes items from the device-wide counter and writes each into both CTAs'
//                queues; every consumer of both CTAs releases the slot on the leader's barrier.

constexpr int P_STAGES = 6;
constexpr uint32_t P_HALF_B = (BN / 2) * BK * 2;             // this CTA's half of the 256 weight rows: 16 KiB
constexpr uint32_t P_STAGE_BYTES = A_BYTES + P_HALF_B;       // 32 KiB
static_assert(P_STAGES * P_STAGE_BYTES == STAGES * STAGE_BYTES, "the pair kernel reuses the single-CTA shared-memory budget");

struct PipeP {
    uint32_t bars, tmem_slot;
    uint8_t* tiles;
    uint8_t* staging;
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8u * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8u * (P_STAGES + s); }
    __device__ __forceinline__ uint32_t acc_full(int b) const { return bars + 8u * (2 * P_STAGES + b); }
    __device__ __forceinline__ uint32_t acc_empty(int b) const { return bars + 8u * (2 * P_STAGES + 2 + b); }
    __device__ __forceinline__ uint32_t sched_full(int i) const { return bars + 8u * (2 * P_STAGES + 5 + i); }
    __device__ __forceinline__ uint32_t sched_empty(int i) const { return bars + 8u * (2 * P_STAGES + 5 + SCHED_Q + i); }
    __device__ __forceinline__ uint32_t sched_item(int i) const { return bars + 8u * (2 * P_STAGES + 5 + 2 * SCHED_Q) + 4u * i; }
};

__device__ __forceinline__ PipeP carve_pair(uint8_t* raw)
{
    PipeP p;
    const uint32_t base = smem_u32(raw);
    const uint32_t pad = (1024u - (base & 1023u)) & 1023u;
    p.tiles = raw + pad;
    p.staging = p.tiles + P_STAGES * P_STAGE_BYTES;
    p.bars = smem_u32(p.staging + EPI_WARPS * STAGING_BYTES);
    p.tmem_slot = p.bars + 8u * (2 * P_STAGES + 4);
    return p;
}

// consumers of a queue slot: the leader's MMA thread, both CTAs' epilogue warps, the peer's producer
constexpr uint32_t P_SCHED_CONSUMERS = 1 + 2 * EPI_WARPS + 1;

struct PairItem {
    int tile0, tile1, n0, e;
};
template <int MODE>
__device__ __forceinline__ PairItem pair_item(const RowsP& p, int item)
{
    constexpr int COLS_PER_ITEM = MODE == MODE_GATEUP ? BN / 2 : BN;
    PairItem w;
    const int pi = item / p.n_col_tiles;
    w.n0 = (item % p.n_col_tiles) * COLS_PER_ITEM;
    w.tile0 = p.pairs[2 * pi];
    w.tile1 = p.pairs[2 * pi + 1];
    w.e = p.tile_expert[w.tile0];
    return w;
}

// This CTA's loads of one work item: its 128 token rows and its half of the weight rows, every k-block, each load
// counted on the LEADER's full barrier.  The leader arms that barrier with both CTAs' bytes.
template <int MODE>
__device__ __forceinline__ bool pair_issue_loads(const PipeP& pipe, const RowsP& p, const PairItem& w, uint32_t rank,
                                                 uint32_t& it, const CUtensorMap* tmA0, const CUtensorMap* tmA1,
                                                 const CUtensorMap* tmB0, const CUtensorMap* tmB1)
{
    const int kb_per_item = (MODE == MODE_DXG ? 2 : 1) * p.kblocks;
    const int my_tile = (rank == 0 || w.tile1 < 0) ? w.tile0 : w.tile1;
    const int row0 = my_tile * BM;
    const int brow = w.e * p.b_rows_per_expert + w.n0;
    for (int kb = 0; kb < kb_per_item; ++kb, ++it) {
        const int s = it % P_STAGES;
        if (it >= (uint32_t)P_STAGES && !mbar_wait_cl(pipe.empty(s), ((it / P_STAGES) - 1) & 1, p.status, ERR_EMPTY_WAIT))
            return false;
        const uint32_t a_dst = smem_u32(pipe.tiles + s * P_STAGE_BYTES), b_dst = a_dst + A_BYTES;
        const uint32_t lead_full = mapa(pipe.full(s), 0);
        if (rank == 0) mbar_expect_tx(pipe.full(s), 2 * P_STAGE_BYTES);
        const bool second = MODE == MODE_DXG && kb >= p.kblocks;
        const int kx = (second ? kb - p.kblocks : kb) * BK;
        tma_load_2d_pair(a_dst, second ? tmA1 : tmA0, kx, row0, lead_full);
        if (MODE == MODE_GATEUP) {
            // the 256 accumulator columns are [128 gate | 128 up]: the leader holds the gate rows, the peer the up rows
            // (tile-major weight copies: block row of (expert, 128-row block, k-block))
            const int y = ((w.e * p.b_row_blocks + (w.n0 >> 7)) * p.b_kb + kb) * 128;
            tma_load_2d_pair(b_dst, rank == 0 ? tmB0 : tmB1, 0, y, lead_full);
        } else if (MODE == MODE_DOWN) {
            const int y = ((w.e * p.b_row_blocks + (w.n0 >> 7) + (int)rank) * p.b_kb + kb) * 128;
            tma_load_2d_pair(b_dst, tmB0, 0, y, lead_full);
        } else {
            tma_load_2d_pair(b_dst, second ? tmB1 : tmB0, kx, brow + (int)rank * (BN / 2), lead_full);
        }
    }
    return true;
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
tc_rows_pair_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                    const __grid_constant__ CUtensorMap tmD0, const __grid_constant__ CUtensorMap tmD1,
                    const __grid_constant__ CUtensorMap tmD2, const RowsP p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, grid_pairs = gridDim.x >> 1;
    const int total_items = *p.n_pairs * p.n_col_tiles;
    if (pair >= total_items) {                 // both CTAs of the pair leave, before any barrier or TMEM use
        if (threadIdx.x == 0 && rank == 0) sched_finish(p.sched, grid_pairs);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const PipeP pipe = carve_pair(smem_raw);

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < P_STAGES; ++s) {
            mbar_init(pipe.full(s), 1);
            mbar_init(pipe.empty(s), 1);
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(pipe.acc_full(b), 1);
            mbar_init(pipe.acc_empty(b), 2 * EPI_WARPS);
        }
#pragma unroll
        for (int i = 0; i < SCHED_Q; ++i) {
            mbar_init(pipe.sched_full(i), 1);
            mbar_init(pipe.sched_empty(i), P_SCHED_CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(pipe.tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync();                            // the peer's barriers exist before anything is sent to them
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(pipe.tmem_slot));

    // a queue slot is released on the leader's barrier, by every consumer of either CTA
    auto release_slot = [&](uint32_t n) {
        const uint32_t bar = pipe.sched_empty(n % SCHED_Q);
        if (rank == 0) mbar_arrive(bar);
        else mbar_arrive_cluster(mapa(bar, 0));
    };
    // the CTA's n-th item (-1: none left); the slot was written by the leader's producer, possibly from the other CTA
    auto consume = [&](uint32_t n) -> int {
        const int slot = n % SCHED_Q;
        if (!mbar_wait_cl(pipe.sched_full(slot), (n / SCHED_Q) & 1, p.status, ERR_SCHED_WAIT)) return -1;
        int item;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(item) : "r"(pipe.sched_item(slot)) : "memory");
        return item;
    };

    if (warp == 0) {
        if (lane == 0 && rank == 0) {
            // leader's producer: hands items to both CTAs, loads its own half of each
            uint32_t it = 0;
            bool ok = true;
            auto publish = [&](uint32_t n, int& item) -> bool {
                const int slot = n % SCHED_Q;
                if (item >= total_items) item = -1;
                if (n >= (uint32_t)SCHED_Q &&
                    !mbar_wait_cl(pipe.sched_empty(slot), ((n / SCHED_Q) - 1) & 1, p.status, ERR_SCHED_WAIT))
                    return false;
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(pipe.sched_item(slot)), "r"(item) : "memory");
                st_cluster_u32(mapa(pipe.sched_item(slot), 1), (uint32_t)item);
                mbar_arrive(pipe.sched_full(slot));
                mbar_arrive_cluster(mapa(pipe.sched_full(slot), 1));       // release at cluster scope: the item is visible
                return true;
            };
            int item = pair;
            ok = publish(0, item);
            for (uint32_t nf = 1; ok && item >= 0; ++nf) {
                const PairItem w = pair_item<MODE>(p, item);
                ok = pair_issue_loads<MODE>(pipe, p, w, 0, it, &tmA0, &tmA1, &tmB0, &tmB1);
                int next = grid_pairs + atomicAdd(p.sched, 1);             // claimed late, as in the single-CTA kernel
                if (ok) ok = publish(nf, next);
                item = next;
            }
            sched_finish(p.sched, grid_pairs);
        } else if (lane == 0) {
            // peer's producer: follows the leader's queue
            uint32_t it = 0;
            for (uint32_t n = 0;; ++n) {
                const int item = consume(n);
                if (item < 0) break;
                release_slot(n);
                const PairItem w = pair_item<MODE>(p, item);
                if (!pair_issue_loads<MODE>(pipe, p, w, 1, it, &tmA0, &tmA1, &tmB0, &tmB1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc(2 * BM, BN, 0, 0);
            const int kb_per_item = (MODE == MODE_DXG ? 2 : 1) * p.kblocks;
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (; ok; ++t) {
                const int item = consume(t);
                if (item < 0) break;
                release_slot(t);
                const uint32_t buf = t & 1u;
                if (t >= 2 && !mbar_wait_cl(pipe.acc_empty(buf), ((t >> 1) - 1) & 1, p.status, ERR_ACC_WAIT)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < kb_per_item; ++kb, ++it) {
                    const int s = it % P_STAGES;
                    if (!mbar_wait_cl(pipe.full(s), (it / P_STAGES) & 1, p.status, ERR_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(pipe.tiles + s * P_STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = make_desc(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = make_desc(b_addr + k * 32, 16, 1024);
                        umma_bf16_pair(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(pipe.empty(s));                 // the stage is free again, in this CTA ...
                    umma_commit_pair(mapa(pipe.empty(s), 1));        // ... and in the peer
                }
                if (ok) {
                    umma_commit_pair(pipe.acc_full(buf));
                    umma_commit_pair(mapa(pipe.acc_full(buf), 1));
                }
            }
        }
    } else {
        const int q = warp & 3, h = (warp - 2) >> 2;
        uint8_t* stage = pipe.staging + (warp - 2) * STAGING_BYTES;
        for (uint32_t t = 0;; ++t) {
            const int item = __shfl_sync(0xffffffffu, consume(t), 0);          // warp-uniform
            if (item < 0) break;
            if (lane == 0) release_slot(t);
            const uint32_t buf = t & 1u;
            const PairItem w = pair_item<MODE>(p, item);
            const bool store = rank == 0 || w.tile1 >= 0;
            const int row_tile = (rank == 0 || w.tile1 < 0) ? w.tile0 : w.tile1;
            const uint32_t acc_empty = rank == 0 ? pipe.acc_empty(buf) : mapa(pipe.acc_empty(buf), 0);
            if (!rows_epilogue<MODE>(p, pipe.acc_full(buf), acc_empty, rank != 0, tmem_base, buf, t, row_tile, w.n0, w.e, q, h,
                                     lane, stage, &tmD0, &tmD1, &tmD2, store))
                break;
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // stores landed before exit
    }
    // neither CTA may leave (or give its TMEM back) while the other can still read its shared memory or signal it
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}
