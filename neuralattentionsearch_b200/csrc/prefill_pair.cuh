// Prefill for a CTA PAIR (thread-block cluster of two, tcgen05 cta_group::2), head_dim 128, group sizes that are a
// multiple of four.  Included by prefill_sm100.cu after its helpers.
//
// A work item = one 128-row query tile x one kv-head x FOUR query heads of its group: CTA c of the pair owns heads
// 2c and 2c + 1 (head slots 0 and 1, as in the single-CTA kernel) with their Q tiles, score / P / O columns and softmax
// warps.  What the pair shares is every K / V tile: each CTA loads only HALF of it -- K rows [64 c, 64 c + 64) (half of the
// N dimension of S = Q.K^T) and V columns [64 c, 64 c + 64) (half of the N dimension of O += P.V) -- and the MMAs are
// issued by the leader CTA with cta_group::2: one instruction runs both SMs' tensor cores, each on its own A operand (its
// Q from shared memory, its P from TMEM) and on the B operand gathered from both CTAs' shared memory.  Per SM that is half
// the L2 -> shared-memory traffic, half the B-operand reads, and a K / V ring that holds five tiles instead of two and a
// half in the same bytes.
//
// Barriers: those the leader's MMA issuers wait on (K / V landed, Q landed, P written, O read) live in the leader and
// collect arrivals from both CTAs (remote arrives, TMA completions addressed to the leader's barrier); what the tensor
// pipe signals (scores ready, O ready, V slot free) is committed to the same barrier in both CTAs.  K slots and Q tiles
// are released locally by each CTA's softmax warps once they see the scores.
#pragma once

namespace nats {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
// TMA load whose completion is counted on a barrier given by its shared::cluster address (the leader's)
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2,
                                                 uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs queued so far have completed
__device__ __forceinline__ void tc_commit2(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
        ::"r"(bar) : "memory");
}
template <int ACC>
__device__ __forceinline__ void mma2_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(ACC) : "memory");
}
template <int ACC>
__device__ __forceinline__ void mma2_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(ACC) : "memory");
}
// Instruction descriptor of the pair: M = 256 (128 rows per CTA)
__host__ __device__ constexpr uint32_t instr_desc2(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

constexpr int kPairSlots = 10;                       // ring slots of half a K or V tile (16 KB at head_dim 128)
constexpr uint32_t kHalfBytes = 64 * 128 * 2;        // half a K tile (64 rows x 128 dims) = half a V tile (128 rows x 64 dims)

struct PairSmem {
    uint8_t q[2][128 * 128 * 2];               // this CTA's two Q tiles
    uint8_t ring[kPairSlots][kHalfBytes];      // this CTA's halves of the K / V tiles, in the order K_0 V_0 K_1 V_1 ...
    uint32_t keep[2][kBitWords];
    uint32_t part[2][kBitWords];
    ItemHeader item[2];
    // leader's copies collect both CTAs (count 2 / 8); the peer's copies of these are unused
    unsigned long long bar_q_full[2], bar_full[kPairSlots], bar_p_full[2][2], bar_o_empty[2];
    // one per CTA, arrivals local or committed to both by the leader
    unsigned long long bar_q_empty[2], bar_empty[kPairSlots], bar_s_full[2], bar_o_full[2];
    unsigned long long bar_list_full[2], bar_list_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int pipe_lock;
};
static_assert(sizeof(PairSmem) <= 232448, "shared memory of the pair kernel");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPrefillThreads, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    constexpr int D = 128;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    PairSmem& sm = *reinterpret_cast<PairSmem*>(smem_raw);
    constexpr int NS = kPairSlots;
    constexpr uint32_t Q_BYTES = 128 * D * 2;
    constexpr uint32_t IDESC_QK = instr_desc2(kTile, false);
    constexpr uint32_t IDESC_PV = instr_desc2(D, true);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cta = cluster_ctarank();              // 0: leader (issues the MMAs), 1: peer
    const bool leader = cta == 0;
    volatile int* abort_flag = &sm.abort_flag;

    if (tid == 0) {
        int bad = (*reinterpret_cast<volatile int32_t*>(p.status) != 0);
        if ((smem_u32(smem_raw) & 1023u) != 0u) {
            atomicCAS(p.status, 0, kErrSmemAlign);
            bad = 1;
        }
        sm.abort_flag = bad;
        sm.pipe_lock = 0;
    }
    __syncthreads();
    // (both CTAs read the same status word; a launch that finds it raised does not start at all)
    if (sm.abort_flag) return;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&sm.bar_full[s]), 2);              // one arrive.expect_tx per CTA
            mbar_init(smem_u32(&sm.bar_empty[s]), 2);             // one arrival per head slot
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(smem_u32(&sm.bar_q_full[h]), 2);
            mbar_init(smem_u32(&sm.bar_q_empty[h]), 1);
            mbar_init(smem_u32(&sm.bar_s_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_p_full[h][0]), 8);         // four softmax warps per CTA
            mbar_init(smem_u32(&sm.bar_p_full[h][1]), 8);
            mbar_init(smem_u32(&sm.bar_o_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_o_empty[h]), 8);
            mbar_init(smem_u32(&sm.bar_list_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_list_empty[h]), leader ? 11 : 9);     // producer, (issuers,) eight softmax warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_q);
        prefetch_tmap(&map_k);
        prefetch_tmap(&map_v);
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(&sm.tmem_base), 512);
        tmem_relinquish2();
        tc_fence_before();
    }
    __syncthreads();
    cluster_sync_all();                                  // both CTAs' barriers exist before anybody arrives remotely
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLow));

    // work items: (batch, kv-head, group of four heads, query tile), heaviest tiles first, dealt round robin to the pairs
    const int n_groups4 = p.nrep / 4;
    const int per_z = p.Nt * p.Hkv * n_groups4;
    const int total = p.total_items;                     // B * Hkv * n_groups4 * Nt
    // round r deals items r * n_pairs ... to the pairs, in alternating direction, so that no pair always gets the heaviest
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    auto my_item = [&](int r) { return r * n_pairs + ((r & 1) ? n_pairs - 1 - pair : pair); };

    if (warp == 3) {
        // =============================== scheduler: item headers, kept-tile bitmaps, this CTA's Q tiles ===============================
        bool ok = true;
        int q_loads = 0;
        const uint64_t pol_q = l2_policy_evict_first();
        const uint32_t qf_leader[2] = {mapa_u32(smem_u32(&sm.bar_q_full[0]), 0), mapa_u32(smem_u32(&sm.bar_q_full[1]), 0)};
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1, use = ic >> 1;
            if (use > 0) ok = warp_wait<kRelaxNs>(smem_u32(&sm.bar_list_empty[slot]), (use - 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const int w = my_item(ic);
            const bool have = w < total;
            int n_kept = 0;
            if (have) {
                const int z = w / per_z, rem = w - z * per_z;
                const int y = rem / p.Nt, x = rem - y * p.Nt;
                const int t = p.Nt - 1 - x;
                const int grp = y % n_groups4, hkv = y / n_groups4;
                const int bh = z * p.Hkv + hkv;
                const int q_lo = p.q_off + t * kTile, q_hi = p.q_off + min(t * kTile + kTile, p.N) - 1;
                const int kt_last = q_hi / kTile;
                const int32_t* tmax = p.tile_max + (size_t)bh * p.Ntk;
                const int32_t* tmin = p.tile_min + (size_t)bh * p.Ntk;
                for (int s0 = 0; s0 <= kt_last; s0 += 32) {
                    const int kt = s0 + lane;
                    const bool keep = kt <= kt_last && tmax[kt] >= q_lo;
                    const bool partial = keep && (kt * kTile + kTile - 1 > q_lo || tmin[kt] < q_hi);
                    const unsigned m = __ballot_sync(0xffffffffu, keep);
                    const unsigned pm = __ballot_sync(0xffffffffu, partial);
                    if (lane == 0) {
                        sm.keep[slot][s0 >> 5] = m;
                        sm.part[slot][s0 >> 5] = pm;
                    }
                    n_kept += __popc(m);
                }
                if (lane == 0) {
                    ItemHeader hd;
                    hd.valid = 1; hd.t = t; hd.b = z; hd.bh = bh; hd.head0 = hkv * p.nrep + grp * 4 + (int)cta * 2;
                    hd.nslots = 2; hd.n_kept = n_kept; hd.pad = 0;
                    sm.item[slot] = hd;
                }
            } else if (lane == 0) {
                sm.item[slot].valid = 0;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.bar_list_full[slot]));
            if (!have) break;
            const ItemHeader hd = sm.item[slot];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (!ok) break;
                if (ic > 0) ok = warp_wait<kRelaxNs>(smem_u32(&sm.bar_q_empty[h]), (ic - 1) & 1, abort_flag, p.status, kErrQ);
                if (!ok) break;
                if (lane == 0) {
                    mbar_expect_tx_cluster(qf_leader[h], Q_BYTES);
                    for (int x = 0; x < 2; ++x)
                        tma_load_3d_pair(smem_u32(&sm.q[h][x * kBoxBytes]), &map_q, qf_leader[h], x * 64, hd.t * kTile,
                                         hd.b * p.Hq + hd.head0 + h, pol_q);
                }
                ++q_loads;
                __syncwarp();
            }
        }
        (void)q_loads;
    } else if (warp == 0) {
        // =============================== producer: this CTA's halves of the K / V tiles ===============================
        uint32_t g = 0;
        const uint64_t pol_kv = l2_policy_evict_last();
        bool ok = true;
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = warp_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            TileWalk walk;
            walk.init(sm.keep[slot], sm.part[slot]);
            for (int j = 0; j < hd.n_kept && ok; ++j) {
                bool partial;
                const int row0 = walk.next(partial) * kTile;
#pragma unroll 1
                for (int kv = 0; kv < 2 && ok; ++kv, ++g) {
                    const int s = g % NS;
                    if (g >= (uint32_t)NS) ok = warp_wait<kRelaxProdNs>(smem_u32(&sm.bar_empty[s]), ((g / NS) & 1) ^ 1, abort_flag, p.status, kErrKvEmpty);
                    if (!ok) break;
                    if (lane == 0) {
                        const uint32_t full_leader = mapa_u32(smem_u32(&sm.bar_full[s]), 0);
                        mbar_expect_tx_cluster(full_leader, kHalfBytes);
                        if (kv == 0) {
                            // K rows [row0 + 64 cta, + 64): two boxes of 64 dims x 64 rows
                            for (int x = 0; x < 2; ++x)
                                tma_load_3d_pair(smem_u32(&sm.ring[s][x * 8192]), &map_k, full_leader, x * 64, row0 + 64 * (int)cta, hd.bh, pol_kv);
                        } else {
                            // V dims [64 cta, + 64) of all 128 rows: one box of 64 dims x 128 rows
                            tma_load_3d_pair(smem_u32(&sm.ring[s][0]), &map_v, full_leader, 64 * (int)cta, row0, hd.bh, pol_kv);
                        }
                    }
                    __syncwarp();
                }
            }
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
    } else if (warp == 1 || warp == 2) {
        if (leader) {
            // =============================== MMA issuers (leader only): warp 1 for head slot 0, warp 2 for head slot 1 ===============================
            const int h = warp - 1;
            constexpr uint32_t H16 = kHalfBytes >> 4, Q16 = Q_BYTES >> 4;
            const uint64_t q_desc = smem_desc(smem_u32(&sm.q[0][0]), 16, 1024) + (uint64_t)(h * Q16);
            const uint64_t k_desc0 = smem_desc(smem_u32(&sm.ring[0][0]), 16, 1024);
            const uint64_t v_desc0 = smem_desc(smem_u32(&sm.ring[0][0]), kBoxBytes, 1024);
            const uint32_t desc_hi = (uint32_t)(q_desc >> 32);
            const uint32_t q_lo = (uint32_t)q_desc, k_lo0 = (uint32_t)k_desc0, v_lo0 = (uint32_t)v_desc0;
            const uint32_t tS = tmem + h * 256, tO = tmem + h * 256 + 128;
            auto issue_qk = [&](int s) {
                // S[256 x 128] = Q[256 x D] . K_j[128 x D]^T; this CTA holds 64 of the 128 K rows: its boxes are 8 KB
                const uint32_t kl = k_lo0 + (uint32_t)s * H16;
                mma2_ss_lo<0>(tS, q_lo, kl, desc_hi, IDESC_QK);
#pragma unroll
                for (int ks = 1; ks < D / 16; ++ks) {
                    const uint32_t qoff = ((ks / 4) * kBoxBytes + (ks % 4) * 32) >> 4;
                    const uint32_t koff = ((ks / 4) * 8192 + (ks % 4) * 32) >> 4;
                    mma2_ss_lo<1>(tS, q_lo + qoff, kl + koff, desc_hi, IDESC_QK);
                }
            };
            auto issue_pv = [&](int s, bool first) {
                // O[256 x D] (+)= P[256 x 128 keys] . V_j[128 x D]; this CTA holds 64 of the D columns, all 128 keys
                const uint32_t vl = v_lo0 + (uint32_t)s * H16;
                if (first) mma2_ts_lo<0>(tO, tS, vl, desc_hi, IDESC_PV);
                else mma2_ts_lo<1>(tO, tS, vl, desc_hi, IDESC_PV);
#pragma unroll
                for (int ks = 1; ks < 8; ++ks) mma2_ts_lo<1>(tO, tS + ks * 8, vl + (uint32_t)(ks * (2048 >> 4)), desc_hi, IDESC_PV);
            };
            uint32_t g = 0, gt = 0, na = 0;
            bool ok = true;
            TR_DECL(8);
#ifdef NATS_TRACE
            unsigned long long tr_lock = 0, tr_pv = 0;
#endif
            for (int ic = 0; ok; ++ic) {
                const int slot = ic & 1;
                ok = warp_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
                if (!ok) break;
                const ItemHeader hd = sm.item[slot];
                if (!hd.valid) break;
                const int n = hd.n_kept;
                ok = warp_wait(smem_u32(&sm.bar_q_full[h]), na & 1, abort_flag, p.status, kErrQ);
                if (ok) ok = warp_wait(smem_u32(&sm.bar_full[g % NS]), (g / NS) & 1, abort_flag, p.status, kErrKvFull);
                if (ok) ok = pipe_acquire(&sm.pipe_lock, lane, abort_flag, p.status);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    issue_qk(g % NS);
                    tc_commit2(smem_u32(&sm.bar_s_full[h]));
                }
                pipe_release(&sm.pipe_lock, lane);
                __syncwarp();
                for (int j = 0; j < n && ok; ++j) {
                    const uint32_t gv = g + 2 * j + 1;
                    const int sv = gv % NS;
                    TR(0);
                    ok = warp_wait(smem_u32(&sm.bar_full[sv]), (gv / NS) & 1, abort_flag, p.status, kErrKvFull);
                    TR(1);
                    const bool more = j + 1 < n;
                    const uint32_t gk = gv + 1;
                    if (ok) ok = warp_wait(smem_u32(&sm.bar_p_full[h][0]), (gt + j) & 1, abort_flag, p.status, kErrPFull);
                    TR(2);
                    if (ok && j == 0 && na > 0) ok = warp_wait(smem_u32(&sm.bar_o_empty[h]), (na - 1) & 1, abort_flag, p.status, kErrOEmpty);
                    TR(3);
                    if (ok) ok = warp_wait(smem_u32(&sm.bar_p_full[h][1]), (gt + j) & 1, abort_flag, p.status, kErrPFull);
                    TR(4);
                    if (ok && more) ok = warp_wait(smem_u32(&sm.bar_full[gk % NS]), (gk / NS) & 1, abort_flag, p.status, kErrKvFull);
                    TR(5);
                    if (ok) ok = pipe_acquire(&sm.pipe_lock, lane, abort_flag, p.status);
                    if (!ok) break;
#ifdef NATS_TRACE
                    { const unsigned long long t_ = clock64(); tr_lock += t_ - tr_t; tr_t = t_; }
#endif
                    tc_fence_after();
                    if (lane == 0) {
                        issue_pv(sv, j == 0);
                        if (!more) tc_commit2(smem_u32(&sm.bar_o_full[h]));
                        tc_commit2(smem_u32(&sm.bar_empty[sv]));           // frees this V slot in both CTAs
#ifdef NATS_TRACE
                        { const unsigned long long t_ = clock64(); tr_pv += t_ - tr_t; tr_t = t_; }
#endif
                        if (more) {
                            issue_qk(gk % NS);
                            tc_commit2(smem_u32(&sm.bar_s_full[h]));
                        }
                    }
                    pipe_release(&sm.pipe_lock, lane);
                    __syncwarp();
                    TR(6);
#ifdef NATS_TRACE
                    tr_acc[7] += 1;
#endif
                }
                g += 2 * n;
                gt += n;
                ++na;
                if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
            }
#ifdef NATS_TRACE
            if (h == 0) { TR_DUMP(16, 8); if (tr_on) { g_trace[24] = tr_lock; g_trace[25] = tr_pv; } }
#endif
        }
    } else {
        // =============================== softmax + epilogue (both CTAs) ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsHigh));
        const int h = (warp - 4) / 4;
        const int row = (warp & 3) * 32 + lane;
        const uint32_t lane_addr = ((uint32_t)((warp & 3) * 32)) << 16;
        const uint32_t tS = tmem + lane_addr + h * 256;
        const uint32_t tO = tmem + lane_addr + h * 256 + 128;
        const float scale = p.scale_log2;
        const bool o_wide = (reinterpret_cast<uintptr_t>(p.o) & 31u) == 0;
        // the barriers the leader's issuer of this head slot waits on
        const uint32_t pf_leader[2] = {mapa_u32(smem_u32(&sm.bar_p_full[h][0]), 0), mapa_u32(smem_u32(&sm.bar_p_full[h][1]), 0)};
        const uint32_t oe_leader = mapa_u32(smem_u32(&sm.bar_o_empty[h]), 0);
        uint32_t gt = 0, na = 0, g = 0;
        const bool releaser = (warp & 3) == 0 && lane == 0;
        bool ok = true;
        TR_DECL(10);
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = warp_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            TR(8);
            const int n = hd.n_kept;
            const int qpos = p.q_off + hd.t * kTile + row;
            const int32_t* lim = p.lim + (size_t)hd.bh * p.Nc;
            float m_ref = -INFINITY, l_sum = 0.f;
            TileWalk walk;
            walk.init(sm.keep[slot], sm.part[slot]);
            for (int j = 0; j < n; ++j, ++gt) {
                bool partial;
                const int k0 = walk.next(partial) * kTile;
                uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
                if (partial) {
                    const int nvis = max(0, min(min(qpos - k0 + 1, p.Nkv - k0), kTile));
#pragma unroll
                    for (int w = 0; w < 4; ++w) bits[w] = range_mask(0, nvis, w);
                    const int c_first = k0 / p.C, c_last = min((k0 + kTile - 1) / p.C, p.Nc - 1);
#pragma unroll 1
                    for (int cc = c_first; cc <= c_last; ++cc) {
                        if (qpos > lim[cc]) {
                            const int lo = max(cc * p.C - k0, 0), hi = min((cc + 1) * p.C - k0, kTile);
#pragma unroll
                            for (int w = 0; w < 4; ++w) bits[w] &= ~range_mask(lo, hi, w);
                        }
                    }
                }
                TR(0);
                ok = warp_wait(smem_u32(&sm.bar_s_full[h]), gt & 1, abort_flag, p.status, kErrSFull);
                if (!ok) break;
                tc_fence_after();
                TR(1);
                if (releaser) {
                    // Q.K^T of tile j has completed in both CTAs: this head slot is done with this CTA's half of K_j and, on the
                    // item's last tile, with its Q tile
                    mbar_arrive(smem_u32(&sm.bar_empty[(g + 2 * j) % NS]));
                    if (j == n - 1) mbar_arrive(smem_u32(&sm.bar_q_empty[h]));
                }
                uint32_t sreg[kTile];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sreg[c * 32]));
                tc_wait_ld();
                TR(2);
                if (partial) {
#pragma unroll
                    for (int i = 0; i < kTile; ++i)
                        if (!((bits[i >> 5] >> (i & 31)) & 1u)) sreg[i] = 0xff800000u;
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < kTile; i += 8) {
                    mx0 = max3(mx0, __uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1]));
                    mx1 = max3(mx1, __uint_as_float(sreg[i + 2]), __uint_as_float(sreg[i + 3]));
                    mx2 = max3(mx2, __uint_as_float(sreg[i + 4]), __uint_as_float(sreg[i + 5]));
                    mx3 = max3(mx3, __uint_as_float(sreg[i + 6]), __uint_as_float(sreg[i + 7]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale;
                float alpha = 1.f;
                bool need = false;
                if (mx > m_ref + kRescaleThreshold) {
                    if (m_ref != -INFINITY) {
                        alpha = ex2(m_ref - mx);
                        l_sum *= alpha;
                        need = true;
                    }
                    m_ref = mx;
                }
                if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld32(tO + c * 32, r);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st32(tO + c * 32, r);
                    }
                }
                const float m_neg = (m_ref == -INFINITY) ? 0.f : -m_ref;
                TR(3);
                const uint64_t scale2 = pack2(scale, scale), mneg2 = pack2(m_neg, m_neg);
                uint64_t ls2 = pack2(0.f, 0.f);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t pk[16];
                        const int base = half * 64 + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const uint64_t x2 = fma2(pack2(__uint_as_float(sreg[base + i]), __uint_as_float(sreg[base + i + 1])), scale2, mneg2);
                            float x0, x1;
                            unpack2(x2, x0, x1);
                            const float p0 = ex2(x0), p1 = ex2(x1);
                            ls2 = add2(ls2, pack2(p0, p1));
                            pk[i / 2] = pack_bf16(p0, p1);
                        }
                        tmem_st16(tS + half * 32 + c * 16, pk);
                    }
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(pf_leader[half]);
#ifdef NATS_TRACE
                    if (half == 0) TR(4); else TR(5);
#endif
                }
                {
                    float a, b;
                    unpack2(ls2, a, b);
                    l_sum += a + b;
                }
            }
            // epilogue
            TR(0);
            if (ok) ok = warp_wait(smem_u32(&sm.bar_o_full[h]), na & 1, abort_flag, p.status, kErrOFull);
            TR(6);
            if (ok) {
                tc_fence_after();
                const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
                const int qi = hd.t * kTile + row;
                __nv_bfloat16* orow = p.o + (((size_t)hd.b * p.Hq + hd.head0 + h) * p.N + qi) * D;
                if (p.lse != nullptr && qi < p.N)
                    p.lse[((size_t)hd.b * p.Hq + hd.head0 + h) * p.N + qi] = l_sum > 0.f ? m_ref + log2f(l_sum) : -INFINITY;
                uint32_t oreg[D];
#pragma unroll
                for (int c = 0; c < D / 32; ++c) tmem_ld32(tO + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&oreg[c * 32]));
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(oe_leader);
                if (qi < p.N) {
#pragma unroll
                    for (int i = 0; i < D; i += 16) {
                        uint32_t w[8];
#pragma unroll
                        for (int x = 0; x < 8; ++x)
                            w[x] = pack_bf16(__uint_as_float(oreg[i + 2 * x]) * inv, __uint_as_float(oreg[i + 2 * x + 1]) * inv);
                        if (o_wide) {
                            st32(orow + i, w);
                        } else {
                            st16(orow + i, make_uint4(w[0], w[1], w[2], w[3]));
                            st16(orow + i + 8, make_uint4(w[4], w[5], w[6], w[7]));
                        }
                    }
                }
            }
            ++na;
            g += 2 * n;
            TR(7);
#ifdef NATS_TRACE
            tr_acc[9] += n;
#endif
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
#ifdef NATS_TRACE
        if (warp == 4) TR_DUMP(0, 10);
#endif
    }
    // ---- teardown: nobody leaves while the other CTA may still touch its shared memory or TMEM ----
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        if (sm.abort_flag) {
            const unsigned long long t0 = global_ns();
            while (global_ns() - t0 < 200000ull) {}
        }
        tc_fence_after();
        tmem_dealloc2(tmem, 512);
    }
}

}  // namespace nats
