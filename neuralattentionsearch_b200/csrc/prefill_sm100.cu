// Role-masked chunked flash-attention prefill for sm_100a: TMA-fed tcgen05.mma with TMEM accumulators.
//
// A work item = one 128-row query tile x one kv-head x up to two query heads of that kv-head's group.  The two heads
// share every K/V tile that is loaded and keep the tensor pipe busy in turns: while the softmax warps of one head
// work on S = Q.K^T in TMEM, the tensor core runs the other head's MMAs.  The kernel is persistent: one CTA per SM
// takes items from a global counter (heaviest query tiles first).
//
//   warp 0      TMA producer: Q of an item, then K and V of every kept KV tile through 2-stage rings
//   warp 3      scheduler: fetches the next item and builds its kept-tile list while the current item runs
//   warps 1,2   MMA issuers of head slot 0 / 1 (one elected lane each): S_h = Q_h.K^T (SS), O_h += P_h.V (TS, P from TMEM)
//   warps 4-7   softmax of head slot 0: one thread per query row, S read with tcgen05.ld, online softmax in
//   warps 8-11  softmax of head slot 1  registers, P written back over S as packed bf16 with tcgen05.st
//
// Which KV tiles are visited comes from the role bitmap: a list of kept tiles is built in shared memory from the
// per-tile max / min row limits (nats_b200_role_prep); tiles without a visible entry are never loaded.  Only tiles
// whose min limit does not cover the whole query tile (and the diagonal) pay for per-element masking.
//
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D); P_h aliases the first 64 columns of S_h.
// Every mbarrier wait is bounded: on a time-out the CTA raises the caller's status word, drains and exits.
#include <cuda.h>

#include "common.cuh"

namespace nats {

constexpr int kPrefillThreads = 384;
constexpr int kStages = 2;
constexpr uint32_t kBoxBytes = 128 * 64 * 2;            // one TMA box: 128 rows x 64 bf16, 128-byte swizzled
#ifndef NATS_RELAX_NS
#define NATS_RELAX_NS 200
#endif
constexpr int kRelaxNs = NATS_RELAX_NS;
#ifndef NATS_RELAX_PROD_NS
#define NATS_RELAX_PROD_NS 0
#endif
constexpr int kRelaxProdNs = NATS_RELAX_PROD_NS;
constexpr float kRescaleThreshold = 8.0f;               // log2 units: O is rescaled only when the row max grows by more
constexpr unsigned long long kWaitLimitNs = 400ull * 1000ull * 1000ull;

enum : int { kErrQ = 1, kErrKFull, kErrVFull, kErrKEmpty, kErrVEmpty, kErrSFull, kErrPFull, kErrOFull, kErrTurn, kErrList, kErrOEmpty };

struct PrefillParams {
    __nv_bfloat16* o;                 // [B,Hq,N,D]
    const int32_t* lim;               // [B,Hkv,Nc]
    const int32_t* tile_max;          // [B,Hkv,Nt]
    const int32_t* tile_min;
    int32_t* status;
    int32_t* work_counter;            // next work item; zero at launch
    int total_items;                  // B * Hkv * n_groups * Nt
    int Hq, Hkv, N, C, Nc, Nt, nrep, n_groups;   // n_groups = ceil(nrep / 2)
    float scale_log2;
};

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false when the wait was given up (by this thread or, earlier, by another one of the CTA).
// With abort_flag == nullptr only the time limit ends the wait (used to drain copies after the CTA has given up).
// RELAX > 0: sleep that many nanoseconds between polls (roles that run ahead of the critical path and should not take
// issue slots from the softmax warps of their scheduler).
template <int RELAX = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
#pragma unroll 1
    for (uint32_t it = 0;; ++it) {
        if (RELAX > 0) __nanosleep(RELAX);
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u) {
            if (abort_flag != nullptr && *abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) {
                if (abort_flag != nullptr) *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; ACC is a compile-time flag so that no predicate has to be computed per MMA
template <int ACC>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets its lane's columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// bits [lo, hi) of a 128-bit row mask that fall into its 32-bit word w
__device__ __forceinline__ uint32_t range_mask(int lo, int hi, int w) {
    const int a = max(lo - 32 * w, 0), b = min(hi - 32 * w, 32);
    if (b <= a) return 0u;
    const uint32_t upto_b = (b >= 32) ? 0xffffffffu : ((1u << b) - 1u);
    return upto_b & ~((1u << a) - 1u);
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---- descriptors ----------------------------------------------------------------------------------
// Shared-memory matrix descriptor of a 128-byte swizzled tile whose rows are 128 bytes (what one TMA box leaves):
// start address >> 4 in [0,14), leading byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46),
// descriptor version 1 in [46,48), swizzle mode 2 (128 B) in [61,64).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulate, bf16 A and B, A K-major, B K-major or MN-major, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// ---- shared memory --------------------------------------------------------------------------------
struct ItemHeader {
    int valid;      // 0: no more work
    int t;          // query tile
    int b, bh;      // batch index, b * Hkv + kv-head
    int head0;      // query head of slot 0
    int nslots;     // 1 or 2 query heads in this item
    int n_kept;     // kept KV tiles
    int pad;
};

template <int D>
struct __align__(1024) PrefillSmem {
    uint8_t q[2][128 * D * 2];             // one tile per head slot; D/64 boxes of 16 KB each
    uint8_t k[kStages][128 * D * 2];
    uint8_t v[kStages][128 * D * 2];
    uint16_t list[2][kMaxTiles];           // kept KV tiles of an item, ascending; bit 15 = needs element masking (double buffered)
    ItemHeader item[2];
    unsigned long long bar_q_full, bar_q_empty;
    unsigned long long bar_k_full[kStages], bar_k_empty[kStages], bar_v_full[kStages], bar_v_empty[kStages];
    unsigned long long bar_s_full[2], bar_p_full[2], bar_o_full[2], bar_o_empty[2], bar_turn[2];
    unsigned long long bar_list_full[2], bar_list_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int kListConsumers = 1 + 2 + 8;     // producer, two issuers, one lane of each of the eight softmax warps

// Persistent kernel: every CTA takes work items (query tile x kv-head x head pair) from a global counter until none is
// left.  Per-item set-up (kept-tile list, Q load) and tear-down (O -> global) overlap the main loops of the neighbouring
// items: warp 3 prepares the list of the next item while the current one runs, the producer streams the next item's K/V
// through the same rings without a bubble, Q of the next item is loaded as soon as the last Q.K^T of the current one
// has completed, and a head's epilogue only delays that head's own chain.
template <int D>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    PrefillSmem<D>& sm = *reinterpret_cast<PrefillSmem<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int NBOX = D / 64;                       // TMA boxes per tile
    constexpr uint32_t TILE_BYTES = NBOX * kBoxBytes;
    constexpr uint32_t IDESC_QK = instr_desc(128, false);
    constexpr uint32_t IDESC_PV = instr_desc(D, true);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    volatile int* abort_flag = &sm.abort_flag;

    if (tid == 0) sm.abort_flag = (*reinterpret_cast<volatile int32_t*>(p.status) != 0);
    __syncthreads();
    if (sm.abort_flag) return;                         // an earlier CTA gave up: do not start (uniform for the CTA)

    // ---- set-up: barriers, TMEM ----
    if (tid == 0) {
        mbar_init(smem_u32(&sm.bar_q_full), 1);
        mbar_init(smem_u32(&sm.bar_q_empty), 2);                   // one commit per MMA issuer
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&sm.bar_k_full[s]), 1);
            mbar_init(smem_u32(&sm.bar_k_empty[s]), 2);
            mbar_init(smem_u32(&sm.bar_v_full[s]), 1);
            mbar_init(smem_u32(&sm.bar_v_empty[s]), 2);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(smem_u32(&sm.bar_s_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_p_full[h]), 128);
            mbar_init(smem_u32(&sm.bar_o_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_o_empty[h]), 128);
            mbar_init(smem_u32(&sm.bar_turn[h]), 1);
            mbar_init(smem_u32(&sm.bar_list_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_list_empty[h]), kListConsumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_q);
        prefetch_tmap(&map_k);
        prefetch_tmap(&map_v);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&sm.tmem_base), 512);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    // Register budget: the softmax warpgroups hold a whole score row per thread (setmaxnreg.inc at the top of their
    // branch), the producer / issuer / scheduler warpgroup needs little and gives registers back.
    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");      // one site for the whole warpgroup

    if (warp == 3) {
        // =============================== scheduler: next work item and its kept-tile list ===============================
        const int per_z = p.Nt * p.Hkv * p.n_groups;
        bool ok = true;
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1, use = ic >> 1;
            if (use > 0) ok = mbar_wait<kRelaxNs>(smem_u32(&sm.bar_list_empty[slot]), (use - 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            int w = 0;
            if (lane == 0) w = atomicAdd(p.work_counter, 1);
            w = __shfl_sync(0xffffffffu, w, 0);
            const bool have = w < p.total_items;
            int n_kept = 0;
            if (have) {
                const int z = w / per_z, rem = w - z * per_z;
                const int y = rem / p.Nt, x = rem - y * p.Nt;
                const int t = p.Nt - 1 - x;                        // heavy (late) query tiles first
                const int grp = y % p.n_groups, hkv = y / p.n_groups;
                const int bh = z * p.Hkv + hkv;
                const int q_lo = t * kTile, q_hi = min(q_lo + kTile, p.N) - 1;
                const int32_t* tmax = p.tile_max + (size_t)bh * p.Nt;
                const int32_t* tmin = p.tile_min + (size_t)bh * p.Nt;
                for (int s0 = 0; s0 <= t; s0 += 32) {              // ordered compaction of the tiles 0..t with a visible entry
                    const int kt = s0 + lane;
                    const bool keep = kt <= t && tmax[kt] >= q_lo;
                    const unsigned m = __ballot_sync(0xffffffffu, keep);
                    if (keep) {
                        const bool partial = kt == t || tmin[kt] < q_hi;
                        sm.list[slot][n_kept + __popc(m & ((1u << lane) - 1u))] = (uint16_t)(kt | (partial ? 0x8000 : 0));
                    }
                    n_kept += __popc(m);
                }
                if (lane == 0) {
                    ItemHeader hd;
                    hd.valid = 1; hd.t = t; hd.b = z; hd.bh = bh; hd.head0 = hkv * p.nrep + grp * 2;
                    hd.nslots = min(2, p.nrep - grp * 2); hd.n_kept = n_kept; hd.pad = 0;
                    sm.item[slot] = hd;
                }
            } else if (lane == 0) {
                sm.item[slot].valid = 0;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.bar_list_full[slot]));
            if (!have) break;
        }
    } else if (warp == 0) {
        // =============================== TMA producer ===============================
        uint32_t g = 0;                                 // tiles pushed through the K / V rings so far (all items)
        uint32_t issued_k = 0, issued_v = 0;
        bool ok = true;
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = mbar_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            // Q of this item may overwrite the previous one once both issuers have committed their last Q.K^T
            if (ic > 0) ok = mbar_wait(smem_u32(&sm.bar_q_empty), (ic - 1) & 1, abort_flag, p.status, kErrQ);
            if (!ok) break;
            if (lane == 0) {
                mbar_expect_tx(smem_u32(&sm.bar_q_full), hd.nslots * TILE_BYTES);
                for (int h = 0; h < hd.nslots; ++h)
                    for (int x = 0; x < NBOX; ++x)
                        tma_load_3d(smem_u32(&sm.q[h][x * kBoxBytes]), &map_q, smem_u32(&sm.bar_q_full), x * 64, hd.t * kTile,
                                    hd.b * p.Hq + hd.head0 + h);
            }
            for (int jt = 0; jt < hd.n_kept && ok; ++jt, ++g) {
                const int kt = sm.list[slot][jt] & 0x7fff;
                const int s = g % kStages;
                const uint32_t ph = (g / kStages) & 1;
                if (g >= kStages) ok = mbar_wait<kRelaxProdNs>(smem_u32(&sm.bar_k_empty[s]), ph ^ 1, abort_flag, p.status, kErrKEmpty);
                if (!ok) break;
                if (lane == 0) {
                    mbar_expect_tx(smem_u32(&sm.bar_k_full[s]), TILE_BYTES);
                    for (int x = 0; x < NBOX; ++x)
                        tma_load_3d(smem_u32(&sm.k[s][x * kBoxBytes]), &map_k, smem_u32(&sm.bar_k_full[s]), x * 64, kt * kTile, hd.bh);
                }
                ++issued_k;
                if (g >= kStages) ok = mbar_wait<kRelaxProdNs>(smem_u32(&sm.bar_v_empty[s]), ph ^ 1, abort_flag, p.status, kErrVEmpty);
                if (!ok) break;
                if (lane == 0) {
                    mbar_expect_tx(smem_u32(&sm.bar_v_full[s]), TILE_BYTES);
                    for (int x = 0; x < NBOX; ++x)
                        tma_load_3d(smem_u32(&sm.v[s][x * kBoxBytes]), &map_v, smem_u32(&sm.bar_v_full[s]), x * 64, kt * kTile, hd.bh);
                }
                ++issued_v;
                __syncwarp();
            }
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
        if (!ok) {
            // given up: let copies that are still in flight land before the shared memory is released
            for (uint32_t x = issued_k > kStages ? issued_k - kStages : 0; x < issued_k; ++x)
                mbar_wait(smem_u32(&sm.bar_k_full[x % kStages]), (x / kStages) & 1, nullptr, p.status, kErrKFull);
            for (uint32_t x = issued_v > kStages ? issued_v - kStages : 0; x < issued_v; ++x)
                mbar_wait(smem_u32(&sm.bar_v_full[x % kStages]), (x / kStages) & 1, nullptr, p.status, kErrVFull);
        }
    } else if (warp == 1 || warp == 2) {
        // =============================== MMA issuers: warp 1 for head slot 0, warp 2 for head slot 1 ===============================
        // Each issuer owns the chain of its head: O_h += P_h.V for tile j, then S_h = Q_h.K^T for tile j+1 (which may only
        // overwrite S_h once the MMA reading P_h from it has been issued).  The two issuers take turns (a token passed
        // through bar_turn): the heads stay half a period apart, so one head's exponentials overlap the other head's MMAs
        // instead of both competing for the same unit at once.  K/V stages and Q are released when both issuers have
        // committed; an issuer whose head slot is empty in an item (odd group size) only keeps the barrier counts going.
        const int h = warp - 1;
        constexpr uint32_t TILE16 = TILE_BYTES >> 4;
        const uint64_t q_desc = smem_desc(smem_u32(&sm.q[0][0]), 16, 1024) + (uint64_t)(h * TILE16);
        const uint64_t k_desc0 = smem_desc(smem_u32(&sm.k[0][0]), 16, 1024);
        const uint64_t v_desc0 = smem_desc(smem_u32(&sm.v[0][0]), kBoxBytes, 1024);
        const uint32_t dS = tmem + h * 128, dO = tmem + 256 + h * 128;
        auto issue_qk = [&](int s) {
            // S_h[128 x 128] = Q_h[128 x D] . K[128 x D]^T : D/16 MMAs of K = 16
            const uint64_t kd = k_desc0 + (uint64_t)(s * TILE16);
            mma_ss<0>(dS, q_desc, kd, IDESC_QK);
#pragma unroll
            for (int ks = 1; ks < D / 16; ++ks) {
                const uint32_t off16 = ((ks / 4) * kBoxBytes + (ks % 4) * 32) >> 4;
                mma_ss<1>(dS, q_desc + off16, kd + off16, IDESC_QK);
            }
        };
        auto issue_pv = [&](int s, bool first) {
            // O_h[128 x D] (+)= P_h[128 x 128] . V[128 x D] : 8 MMAs of K = 16; V is MN-major (D contiguous)
            const uint64_t vd = v_desc0 + (uint64_t)(s * TILE16);
            mma_ts(dO, dS, vd, IDESC_PV, first ? 0u : 1u);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) mma_ts(dO, dS + ks * 8, vd + (uint64_t)(ks * (2048 >> 4)), IDESC_PV, 1u);
        };
        uint32_t g = 0;          // tiles through the K / V rings (all items, both issuers count alike)
        uint32_t gh = 0;         // tiles of this head (items in which its slot is used)
        uint32_t na = 0;         // items in which this head's slot was used
        uint32_t turns = 0;      // turns taken in two-head items
        bool ok = true;
        auto take_turn = [&]() {
            // issuer 0 follows issuer 1's previous turn, issuer 1 follows issuer 0's turn of the same number
            if (h == 0) return turns == 0 ? true : mbar_wait(smem_u32(&sm.bar_turn[0]), (turns - 1) & 1, abort_flag, p.status, kErrTurn);
            return mbar_wait(smem_u32(&sm.bar_turn[1]), turns & 1, abort_flag, p.status, kErrTurn);
        };
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = mbar_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            const int n = hd.n_kept;
            const bool active = h < hd.nslots, two = hd.nslots == 2;
            if (active) ok = mbar_wait(smem_u32(&sm.bar_q_full), ic & 1, abort_flag, p.status, kErrQ);
            // ---- first tile: S_h = Q_h.K^T ----
            if (ok) ok = mbar_wait(smem_u32(&sm.bar_k_full[g % kStages]), (g / kStages) & 1, abort_flag, p.status, kErrKFull);
            if (ok && active && two) ok = take_turn();
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                if (active) {
                    issue_qk(g % kStages);
                    tc_commit(smem_u32(&sm.bar_s_full[h]));
                }
                tc_commit(smem_u32(&sm.bar_k_empty[g % kStages]));
                if (n == 1) tc_commit(smem_u32(&sm.bar_q_empty));
                if (active && two) mbar_arrive(smem_u32(&sm.bar_turn[1 - h]));
            }
            if (active && two) ++turns;
            __syncwarp();
            // ---- tiles ----
            for (int jt = 0; jt < n && ok; ++jt, ++g) {
                const int s = g % kStages;
                const uint32_t ph = (g / kStages) & 1;
                const bool has_next = jt + 1 < n;
                const int sn = (g + 1) % kStages;
                const uint32_t phn = ((g + 1) / kStages) & 1;
                ok = mbar_wait(smem_u32(&sm.bar_v_full[s]), ph, abort_flag, p.status, kErrVFull);
                if (ok && has_next) ok = mbar_wait(smem_u32(&sm.bar_k_full[sn]), phn, abort_flag, p.status, kErrKFull);
                if (ok && active) ok = mbar_wait(smem_u32(&sm.bar_p_full[h]), gh & 1, abort_flag, p.status, kErrPFull);
                // the first P.V of an item overwrites O_h: the previous item's epilogue must have read it
                if (ok && active && jt == 0 && na > 0) ok = mbar_wait(smem_u32(&sm.bar_o_empty[h]), (na - 1) & 1, abort_flag, p.status, kErrOEmpty);
                if (ok && active && two) ok = take_turn();
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    if (active) {
                        issue_pv(s, jt == 0);
                        if (!has_next) tc_commit(smem_u32(&sm.bar_o_full[h]));
                    }
                    tc_commit(smem_u32(&sm.bar_v_empty[s]));
                    if (has_next) {
                        if (active) {
                            issue_qk(sn);
                            tc_commit(smem_u32(&sm.bar_s_full[h]));
                        }
                        tc_commit(smem_u32(&sm.bar_k_empty[sn]));
                        if (jt + 2 == n) tc_commit(smem_u32(&sm.bar_q_empty));      // that was the last Q.K^T of the item
                    }
                    if (active && two) mbar_arrive(smem_u32(&sm.bar_turn[1 - h]));
                }
                if (active && two) ++turns;
                if (active) ++gh;
                __syncwarp();
            }
            if (active) ++na;
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
    } else if (warp >= 4) {
        // =============================== softmax + epilogue ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        const int h = (warp - 4) / 4;                    // head slot
        const int row = (warp & 3) * 32 + lane;          // query row inside the tile == TMEM lane
        const uint32_t lane_addr = ((uint32_t)((warp & 3) * 32)) << 16;
        const uint32_t tS = tmem + lane_addr + h * 128;
        const uint32_t tO = tmem + lane_addr + 256 + h * 128;
        const float scale = p.scale_log2;
        uint32_t gh = 0, na = 0;                         // tiles / items of this head so far
        bool ok = true;
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = mbar_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            if (h < hd.nslots) {
                const int n_kept = hd.n_kept;
                const int q_lo = hd.t * kTile;
                const int qi = q_lo + row;                       // query token index
                const int32_t* lim = p.lim + (size_t)hd.bh * p.Nc;
                float m_ref = -INFINITY, l_sum = 0.f;
                for (int jt = 0; jt < n_kept; ++jt, ++gh) {
                    const int entry = sm.list[slot][jt];
                    const int kt = entry & 0x7fff;
                    const bool partial = (entry & 0x8000) != 0;
                    // visibility bits of this row for the 128 columns of a tile that is not fully visible
                    uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
                    if (partial) {
                        // columns this row may see: the causal prefix (and nothing past N), minus every chunk whose row limit is below it
                        const int k0 = kt * kTile;
                        const int nvis = max(0, min(min(qi - k0 + 1, p.N - k0), kTile));
#pragma unroll
                        for (int w = 0; w < 4; ++w) bits[w] = range_mask(0, nvis, w);
                        const int c_first = k0 / p.C, c_last = min((k0 + kTile - 1) / p.C, p.Nc - 1);
#pragma unroll 1
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            if (qi > lim[cc]) {
                                const int lo = max(cc * p.C - k0, 0), hi = min((cc + 1) * p.C - k0, kTile);
#pragma unroll
                                for (int w = 0; w < 4; ++w) bits[w] &= ~range_mask(lo, hi, w);
                            }
                        }
                    }
                    ok = mbar_wait(smem_u32(&sm.bar_s_full[h]), gh & 1, abort_flag, p.status, kErrSFull);
                    if (!ok) break;
                    tc_fence_after();
                    // the whole score row of this thread in registers: four loads in flight, one wait
                    uint32_t sreg[128];
                    tmem_ld32(tS + 0, *reinterpret_cast<uint32_t(*)[32]>(&sreg[0]));
                    tmem_ld32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&sreg[32]));
                    tmem_ld32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&sreg[64]));
                    tmem_ld32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&sreg[96]));
                    tc_wait_ld();
                    if (partial) {
#pragma unroll
                        for (int i = 0; i < 128; ++i)
                            if (!((bits[i >> 5] >> (i & 31)) & 1u)) sreg[i] = 0xff800000u;      // -inf: exp2 gives exactly 0
                    }
                    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 128; i += 4) {
                        mx0 = fmaxf(mx0, __uint_as_float(sreg[i]));
                        mx1 = fmaxf(mx1, __uint_as_float(sreg[i + 1]));
                        mx2 = fmaxf(mx2, __uint_as_float(sreg[i + 2]));
                        mx3 = fmaxf(mx3, __uint_as_float(sreg[i + 3]));
                    }
                    const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale;       // scale > 0
                    // online softmax with lazy rescaling: the reference maximum only moves when the row max grew by > threshold
                    float alpha = 1.f;
                    bool need = false;
                    if (mx > m_ref + kRescaleThreshold) {           // also true for the first visible tile (m_ref = -inf)
                        if (m_ref != -INFINITY) {                   // a row without visible entries so far has O = 0, l = 0
                            alpha = ex2(m_ref - mx);
                            l_sum *= alpha;
                            need = true;
                        }
                        m_ref = mx;
                    }
                    if (jt > 0 && __any_sync(0xffffffffu, need)) {
                        // O_h of the previous tiles is complete (the commit behind S_h covers every earlier MMA): rescale it
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
                    // P = exp2(S * scale - m), row sum in fp32, P packed to bf16 over the first 64 columns of S_h
                    float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = ex2(fmaf(__uint_as_float(sreg[c * 32 + i]), scale, m_neg));
                            const float p1 = ex2(fmaf(__uint_as_float(sreg[c * 32 + i + 1]), scale, m_neg));
                            ls0 += p0;
                            ls1 += p1;
                            pk[i / 2] = pack_bf16(p0, p1);
                        }
                        tmem_st16(tS + c * 16, pk);
                    }
                    l_sum += ls0 + ls1;
                    tc_wait_st();
                    tc_fence_before();
                    mbar_arrive(smem_u32(&sm.bar_p_full[h]));
                }
                // epilogue: O / l -> bf16 -> global; O_h is handed back to the issuer as soon as it sits in registers
                if (ok && n_kept > 0) ok = mbar_wait(smem_u32(&sm.bar_o_full[h]), na & 1, abort_flag, p.status, kErrOFull);
                if (ok && n_kept > 0) {
                    tc_fence_after();
                    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
                    __nv_bfloat16* orow = p.o + (((size_t)hd.b * p.Hq + hd.head0 + h) * p.N + qi) * D;
                    uint32_t oreg[D];
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) tmem_ld32(tO + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&oreg[c * 32]));
                    tc_wait_ld();
                    tc_fence_before();
                    mbar_arrive(smem_u32(&sm.bar_o_empty[h]));
                    if (qi < p.N) {
#pragma unroll
                        for (int i = 0; i < D; i += 8) {
                            uint4 w;
                            w.x = pack_bf16(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv);
                            w.y = pack_bf16(__uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv);
                            w.z = pack_bf16(__uint_as_float(oreg[i + 4]) * inv, __uint_as_float(oreg[i + 5]) * inv);
                            w.w = pack_bf16(__uint_as_float(oreg[i + 6]) * inv, __uint_as_float(oreg[i + 7]) * inv);
                            st16(orow + i, w);
                        }
                    }
                }
                ++na;
            }
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
    }
    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (sm.abort_flag) {
            // MMAs may still be running: give them time before the accumulator columns are released
            const unsigned long long t0 = global_ns();
            while (global_ns() - t0 < 200000ull) {}
        }
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = (EncodeTiledFn)ptr;
    return fn;
}

// [heads, N, D] bf16 viewed as a 3-D tensor (D innermost); box = 64 x 128 x 1 with 128-byte swizzle; rows past N read zero
static int make_map(CUtensorMap* map, const void* base, int heads, int N, int D) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(NATS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)heads};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)N * D * 2};
    cuuint32_t box[3] = {64, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NATS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return NATS_OK;
}

struct PrefillWs { size_t lim, tmax, tmin, counter, total; };
static PrefillWs prefill_ws(int B, int Hkv, int N, int C) {
    PrefillWs w;
    const size_t Nc = cdiv(N, C), Nt = cdiv(N, kTile);
    w.lim = 0;
    w.tmax = align_up((size_t)B * Hkv * Nc * 4, 256);
    w.tmin = w.tmax + align_up((size_t)B * Hkv * Nt * 4, 256);
    w.counter = w.tmin + align_up((size_t)B * Hkv * Nt * 4, 256);
    w.total = w.counter + 256;
    return w;
}

template <int D>
static int launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p,
                          int B, cudaStream_t st) {
    const size_t smem = sizeof(PrefillSmem<D>) + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        NATS_CHECK_CUDA(cudaFuncSetAttribute(prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    int dev = 0, sms = 0;
    NATS_CHECK_CUDA(cudaGetDevice(&dev));
    NATS_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    NATS_CHECK_CUDA(cudaMemsetAsync(p.work_counter, 0, sizeof(int32_t), st));
    const int grid = p.total_items < sms ? p.total_items : sms;      // one persistent CTA per SM
    (void)B;
    prefill_kernel<D><<<grid, kPrefillThreads, smem, st>>>(mq, mk, mv, p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

}  // namespace nats

using namespace nats;

extern "C" __attribute__((visibility("default"))) size_t nats_b200_prefill_workspace_bytes(int B, int Hkv, int N, int C) {
    if (B <= 0 || Hkv <= 0 || N <= 0 || C <= 0) return 0;
    return prefill_ws(B, Hkv, N, C).total;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_prefill_fwd(const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
                                     int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale,
                                     void* d_workspace, size_t workspace_bytes, int64_t* d_kept_tiles, int32_t* d_status,
                                     void* stream) {
    NATS_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && N > 0 && Hq % Hkv == 0, "bad shape B=%d Hq=%d Hkv=%d N=%d", B, Hq, Hkv, N);
    NATS_CHECK_ARG(C > 0 && SW > 0 && SW % C == 0, "sliding window %d must be a positive multiple of the chunk size %d", SW, C);
    NATS_CHECK_ARG(d_q && d_k && d_v && d_o && d_roles && d_workspace && d_status, "null pointer");
    NATS_CHECK_ARG(((uintptr_t)d_q | (uintptr_t)d_k | (uintptr_t)d_v | (uintptr_t)d_o | (uintptr_t)d_workspace) % 16 == 0,
                   "q, k, v, o and the workspace must be 16-byte aligned");
    NATS_CHECK_ARG(sm_scale > 0.f, "sm_scale must be positive");
    if (D != 64 && D != 128) return fail(NATS_ERR_UNSUPPORTED, "prefill supports head_dim 64 and 128, got %d", D);
    NATS_CHECK_ARG(N <= kMaxTiles * kTile, "N = %d exceeds the prefill limit %d", N, kMaxTiles * kTile);
    NATS_CHECK_ARG((long long)B <= 65535 && (long long)Hkv * ((Hq / Hkv + 1) / 2) <= 65535, "grid too large");
    const PrefillWs w = prefill_ws(B, Hkv, N, C);
    if (workspace_bytes < w.total)
        return fail(NATS_ERR_WORKSPACE, "prefill workspace: %zu bytes given, %zu needed", workspace_bytes, w.total);
    uint8_t* ws = (uint8_t*)d_workspace;
    int32_t* lim = (int32_t*)(ws + w.lim);
    int32_t* tmax = (int32_t*)(ws + w.tmax);
    int32_t* tmin = (int32_t*)(ws + w.tmin);
    if (int rc = nats_b200_role_prep(d_roles, B, Hkv, N, C, SW, lim, tmax, tmin, d_kept_tiles, stream)) return rc;
    CUtensorMap mq, mk, mv;
    if (int rc = make_map(&mq, d_q, B * Hq, N, D)) return rc;
    if (int rc = make_map(&mk, d_k, B * Hkv, N, D)) return rc;
    if (int rc = make_map(&mv, d_v, B * Hkv, N, D)) return rc;
    PrefillParams p;
    p.o = (__nv_bfloat16*)d_o; p.lim = lim; p.tile_max = tmax; p.tile_min = tmin; p.status = d_status;
    p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.C = C; p.Nc = cdiv(N, C); p.Nt = cdiv(N, kTile);
    p.nrep = Hq / Hkv; p.n_groups = (p.nrep + 1) / 2;
    p.work_counter = (int32_t*)(ws + w.counter);
    const long long items = (long long)B * Hkv * p.n_groups * p.Nt;
    NATS_CHECK_ARG(items <= 0x7fffffffLL - 65536, "too many work items (%lld)", items);
    p.total_items = (int)items;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    if (D == 64) return launch_prefill<64>(mq, mk, mv, p, B, (cudaStream_t)stream);
    return launch_prefill<128>(mq, mk, mv, p, B, (cudaStream_t)stream);
}

// =================================================================================================
// Prefill without any allocation by the caller or by this library
// =================================================================================================
namespace nats {

constexpr size_t kStaticScratchBytes = 1u << 20;   // 1 MiB per GPU that loads the library, held until the process exits
constexpr int kMaxDevices = 64;

// Scratch for the role metadata (row limits and per-tile max / min limits) of nats_b200_prefill_fwd_static.
// In host code this name is only a stand-in for the symbol: the device address is obtained once per device below.
static __device__ __align__(256) uint8_t g_prefill_scratch[kStaticScratchBytes];
static void* g_prefill_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the current device; looked up on the first call per device.
static int static_scratch(void** out) {
    int dev = -1;
    NATS_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(NATS_ERR_UNSUPPORTED, "device index %d is outside [0, %d)", dev, kMaxDevices);
    if (g_prefill_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_prefill_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(NATS_ERR_CUDA, "cudaGetSymbolAddress(g_prefill_scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
        g_prefill_scratch_addr[dev] = ptr;
    }
    *out = g_prefill_scratch_addr[dev];
    return NATS_OK;
}

}  // namespace nats

extern "C" __attribute__((visibility("default"))) size_t nats_b200_prefill_static_scratch_bytes(void) {
    return nats::kStaticScratchBytes;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_prefill_fwd_static(
    const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
    int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale,
    int64_t* d_kept_tiles, int32_t* d_status, void* stream) {
    if (B <= 0 || Hkv <= 0 || N <= 0 || C <= 0) return fail(NATS_ERR_INVALID_ARG, "bad shape B=%d Hkv=%d N=%d C=%d", B, Hkv, N, C);
    const size_t need = nats_b200_prefill_workspace_bytes(B, Hkv, N, C);
    if (need > nats::kStaticScratchBytes)
        return fail(NATS_ERR_WORKSPACE,
                    "this shape needs %zu bytes of role metadata, the built-in scratch holds %zu: use nats_b200_prefill_fwd "
                    "with a caller-provided workspace", need, (size_t)nats::kStaticScratchBytes);
    void* scratch = nullptr;
    if (int rc = nats::static_scratch(&scratch)) return rc;
    return nats_b200_prefill_fwd(d_q, d_k, d_v, d_o, d_roles, B, Hq, Hkv, N, D, C, SW, sm_scale, scratch,
                                 nats::kStaticScratchBytes, d_kept_tiles, d_status, stream);
}

