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
#ifndef NATS_REGS_LOW
#define NATS_REGS_LOW 72
#endif
#ifndef NATS_REGS_HIGH
#define NATS_REGS_HIGH 216
#endif
// setmaxnreg split: 128 * low + 256 * high must not exceed the 384 * 168 registers of the launch
constexpr int kRegsLow = NATS_REGS_LOW, kRegsHigh = NATS_REGS_HIGH;
static_assert(128 * kRegsLow + 256 * kRegsHigh <= 384 * 168, "setmaxnreg budget");
#ifndef NATS_PINGPONG
#define NATS_PINGPONG 1
#endif
constexpr bool kPingPong = NATS_PINGPONG != 0;   // the two heads' warps that share a scheduler take turns on the MUFU pipe
constexpr int kStages = 4;                              // K/V ring depth, in 64-row sub-tiles
constexpr int kSub = 64;                                // key columns per sub-tile (two per kept 128-column tile)
constexpr uint32_t kQBoxBytes = 128 * 64 * 2;           // one TMA box of Q: 128 rows x 64 bf16, 128-byte swizzled
constexpr uint32_t kKvBoxBytes = kSub * 64 * 2;         // one TMA box of K or V: 64 rows x 64 bf16
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

enum : int { kErrQ = 1, kErrKFull, kErrVFull, kErrKEmpty, kErrVEmpty, kErrSFull, kErrPFull, kErrOFull, kErrTurn, kErrList, kErrOEmpty, kErrPvDone, kErrMufu };

struct PrefillParams {
    __nv_bfloat16* o;                 // [B,Hq,N,D]
    float* lse;                       // [B,Hq,N] or nullptr: log2 of the row's sum of exp2(score * scale * log2 e)
    const int32_t* lim;               // [B,Hkv,Nc]: last query POSITION that may see KV chunk c
    const int32_t* tile_max;          // [B,Hkv,Ntk]: max / min of lim over the chunks of a 128-row KV tile
    const int32_t* tile_min;
    int32_t* status;
    int32_t* work_counter;            // next work item; zero at launch
    int total_items;                  // B * Hkv * n_groups * Nt
    // N query rows; query row i sits at position q_off + i of the KV sequence of Nkv rows (a first call has q_off = 0 and
    // Nkv = N; a call over an existing cache attends to the cache rows in front of its own tokens).
    // Nc / Ntk: chunks / 128-row tiles of the KV sequence, Nt: query tiles.
    int Hq, Hkv, N, Nkv, q_off, C, Nc, Nt, Ntk, nrep, n_groups;   // n_groups = ceil(nrep / 2)
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
// issue slots from the softmax warps of their scheduler).  Every lane of a waiting warp polls: letting one lane poll and
// broadcast the result was measured 25 % slower for the whole kernel.
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
    int n_kept;     // kept 128-column KV tiles (each is processed as two 64-column sub-tiles)
    int pad;
};

template <int D>
struct __align__(1024) PrefillSmem {
    uint8_t q[2][128 * D * 2];             // one tile per head slot; D/64 boxes of 16 KB each
    uint8_t kv[kStages][2][kSub * D * 2];  // per stage: K sub-tile, V sub-tile; D/64 boxes of 8 KB each
    uint16_t list[2][kMaxTiles];           // kept KV tiles of an item, ascending; bit 15 = needs element masking (double buffered)
    ItemHeader item[2];
    unsigned long long bar_q_full, bar_q_empty;
    unsigned long long bar_kv_full[kStages], bar_kv_empty[kStages];
    unsigned long long bar_s_full[2][2], bar_p_full[2][2], bar_pv_done[2], bar_o_full[2], bar_o_empty[2];
    unsigned long long bar_list_full[2], bar_list_empty[2];
    unsigned long long bar_mufu[2][4];     // [head slot][warp quarter]: permission to run the exponentials
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int kListConsumers = 1 + 2 + 8;     // producer, two issuers, one lane of each of the eight softmax warps

// Persistent kernel: every CTA takes work items (query tile x kv-head x head pair) from a global counter until none is
// left.  Per-item set-up (kept-tile list, Q load) and tear-down (O -> global) overlap the main loops of the neighbouring
// items: warp 3 prepares the list of the next item while the current one runs, the producer streams the next item's K/V
// through the same ring without a bubble, Q of the next item is loaded as soon as the last Q.K^T of the current one
// has completed, and a head's epilogue only delays that head's own chain.
//
// A kept 128-column KV tile is processed as two 64-column sub-tiles, and every head has TWO score buffers in TMEM
// (S_a, S_b: 64 columns each) next to its 128-column O accumulator.  S = Q.K^T of sub-tile u+1 is therefore computed
// while the softmax warps still work on sub-tile u: the softmax of a head runs back to back and only O += P.V waits for
// it, so the tensor pipe is kept busy by two independent chains instead of being stalled by one softmax latency per tile.
template <int D>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    PrefillSmem<D>& sm = *reinterpret_cast<PrefillSmem<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int NBOX = D / 64;                       // TMA boxes per tile
    constexpr uint32_t Q_BYTES = NBOX * kQBoxBytes;    // one Q tile (128 rows)
    constexpr uint32_t SUB_BYTES = NBOX * kKvBoxBytes; // one K or V sub-tile (64 rows)
    constexpr uint32_t IDESC_QK = instr_desc(kSub, false);
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
            mbar_init(smem_u32(&sm.bar_kv_full[s]), 1);
            mbar_init(smem_u32(&sm.bar_kv_empty[s]), 2);
        }
        for (int h = 0; h < 2; ++h) {
            for (int x = 0; x < 2; ++x) {
                mbar_init(smem_u32(&sm.bar_s_full[h][x]), 1);
                mbar_init(smem_u32(&sm.bar_p_full[h][x]), 4);              // one arrival per softmax warp
            }
            mbar_init(smem_u32(&sm.bar_pv_done[h]), 1);
            mbar_init(smem_u32(&sm.bar_o_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_o_empty[h]), 4);
            mbar_init(smem_u32(&sm.bar_list_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_list_empty[h]), kListConsumers);
            for (int x = 0; x < 4; ++x) mbar_init(smem_u32(&sm.bar_mufu[h][x]), 1);
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

    // Register budget: the softmax warpgroups get more registers (setmaxnreg.inc at the top of their branch), the
    // producer / issuer / scheduler warpgroup needs little and gives registers back.
    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLow));      // one site for the whole warpgroup

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
                // positions of the first and last query row of the tile; KV tiles up to the one holding the last row
                const int q_lo = p.q_off + t * kTile, q_hi = p.q_off + min(t * kTile + kTile, p.N) - 1;
                const int kt_last = q_hi / kTile;
                const int32_t* tmax = p.tile_max + (size_t)bh * p.Ntk;
                const int32_t* tmin = p.tile_min + (size_t)bh * p.Ntk;
                for (int s0 = 0; s0 <= kt_last; s0 += 32) {        // ordered compaction of the tiles 0..kt_last with a visible entry
                    const int kt = s0 + lane;
                    const bool keep = kt <= kt_last && tmax[kt] >= q_lo;
                    const unsigned m = __ballot_sync(0xffffffffu, keep);
                    if (keep) {
                        // element masking is needed where the causal edge or a chunk's row limit cuts through the tile
                        const bool partial = kt * kTile + kTile - 1 > q_lo || tmin[kt] < q_hi;
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
        uint32_t g = 0;                                 // sub-tiles pushed through the K/V ring so far (all items)
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
                mbar_expect_tx(smem_u32(&sm.bar_q_full), hd.nslots * Q_BYTES);
                for (int h = 0; h < hd.nslots; ++h)
                    for (int x = 0; x < NBOX; ++x)
                        tma_load_3d(smem_u32(&sm.q[h][x * kQBoxBytes]), &map_q, smem_u32(&sm.bar_q_full), x * 64, hd.t * kTile,
                                    hd.b * p.Hq + hd.head0 + h);
            }
            for (int u = 0; u < 2 * hd.n_kept && ok; ++u, ++g) {
                const int kt = sm.list[slot][u >> 1] & 0x7fff;
                const int row0 = kt * kTile + (u & 1) * kSub;
                const int s = g % kStages;
                const uint32_t ph = (g / kStages) & 1;
                if (g >= kStages) ok = mbar_wait<kRelaxProdNs>(smem_u32(&sm.bar_kv_empty[s]), ph ^ 1, abort_flag, p.status, kErrKEmpty);
                if (!ok) break;
                if (lane == 0) {
                    mbar_expect_tx(smem_u32(&sm.bar_kv_full[s]), 2 * SUB_BYTES);
                    for (int x = 0; x < NBOX; ++x)
                        tma_load_3d(smem_u32(&sm.kv[s][0][x * kKvBoxBytes]), &map_k, smem_u32(&sm.bar_kv_full[s]), x * 64, row0, hd.bh);
                    for (int x = 0; x < NBOX; ++x)
                        tma_load_3d(smem_u32(&sm.kv[s][1][x * kKvBoxBytes]), &map_v, smem_u32(&sm.bar_kv_full[s]), x * 64, row0, hd.bh);
                }
                __syncwarp();
            }
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
        if (!ok) {
            // given up: let copies that are still in flight land before the shared memory is released
            for (uint32_t x = g > kStages ? g - kStages : 0; x < g; ++x)
                mbar_wait(smem_u32(&sm.bar_kv_full[x % kStages]), (x / kStages) & 1, nullptr, p.status, kErrKFull);
        }
    } else if (warp == 1 || warp == 2) {
        // =============================== MMA issuers: warp 1 for head slot 0, warp 2 for head slot 1 ===============================
        // Per head and 64-column sub-tile u:  S[u & 1] = Q_h.K_u^T  (issued two sub-tiles ahead of the softmax) and
        // O_h += P_u.V_u once the softmax warps have written P_u over S[u & 1].  S[u & 1] is overwritten by sub-tile u + 2
        // only after the MMA that reads P_u has been issued (same thread, so the tensor pipe keeps the order).
        // A K/V stage is released when both issuers have committed its P.V; an issuer whose head slot is empty in an item
        // (odd group size) only keeps the barrier counts going.
        const int h = warp - 1;
        constexpr uint32_t Q16 = Q_BYTES >> 4, SUB16 = SUB_BYTES >> 4, STAGE16 = (2 * SUB_BYTES) >> 4;
        const uint64_t q_desc = smem_desc(smem_u32(&sm.q[0][0]), 16, 1024) + (uint64_t)(h * Q16);
        const uint64_t k_desc0 = smem_desc(smem_u32(&sm.kv[0][0][0]), 16, 1024);
        const uint64_t v_desc0 = smem_desc(smem_u32(&sm.kv[0][1][0]), kKvBoxBytes, 1024);
        const uint32_t tS = tmem + h * 256, tO = tmem + h * 256 + 128;
        auto issue_qk = [&](int s, int buf) {
            // S[buf][128 x 64] = Q_h[128 x D] . K_u[64 x D]^T : D/16 MMAs of K = 16
            const uint64_t kd = k_desc0 + (uint64_t)(s * STAGE16);
            const uint32_t dS = tS + buf * kSub;
            mma_ss<0>(dS, q_desc, kd, IDESC_QK);
#pragma unroll
            for (int ks = 1; ks < D / 16; ++ks) {
                const uint32_t qoff = ((ks / 4) * kQBoxBytes + (ks % 4) * 32) >> 4;
                const uint32_t koff = ((ks / 4) * kKvBoxBytes + (ks % 4) * 32) >> 4;
                mma_ss<1>(dS, q_desc + qoff, kd + koff, IDESC_QK);
            }
        };
        auto issue_pv = [&](int s, int buf, bool first) {
            // O_h[128 x D] (+)= P_u[128 x 64] . V_u[64 x D] : 4 MMAs of K = 16; V is MN-major (D contiguous)
            const uint64_t vd = v_desc0 + (uint64_t)(s * STAGE16);
            const uint32_t aP = tS + buf * kSub;
            mma_ts(tO, aP, vd, IDESC_PV, first ? 0u : 1u);
#pragma unroll
            for (int ks = 1; ks < kSub / 16; ++ks) mma_ts(tO, aP + ks * 8, vd + (uint64_t)(ks * (2048 >> 4)), IDESC_PV, 1u);
        };
        (void)SUB16;
        uint32_t g = 0;          // sub-tiles through the K/V ring (all items, both issuers count alike)
        uint32_t gu = 0;         // sub-tiles of this head (items in which its slot is used); even at every item start
        uint32_t na = 0;         // items in which this head's slot was used
        bool ok = true;
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = mbar_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            const int n2 = 2 * hd.n_kept;
            const bool active = h < hd.nslots;
            if (active) ok = mbar_wait(smem_u32(&sm.bar_q_full), ic & 1, abort_flag, p.status, kErrQ);
            // ---- the first two score buffers ----
            for (int x = 0; x < 2 && ok; ++x) {
                const uint32_t gx = g + x;
                ok = mbar_wait(smem_u32(&sm.bar_kv_full[gx % kStages]), (gx / kStages) & 1, abort_flag, p.status, kErrKFull);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    if (active) {
                        issue_qk(gx % kStages, x);
                        tc_commit(smem_u32(&sm.bar_s_full[h][x]));
                    }
                    if (x == 1 && n2 == 2) tc_commit(smem_u32(&sm.bar_q_empty));
                }
                __syncwarp();
            }
            // ---- sub-tiles ----
            for (int u = 0; u < n2 && ok; ++u) {
                const uint32_t gs = g + u;
                const int s = gs % kStages, buf = u & 1;
                const bool more = u + 2 < n2;
                if (active) {
                    ok = mbar_wait(smem_u32(&sm.bar_p_full[h][buf]), ((gu + u) >> 1) & 1, abort_flag, p.status, kErrPFull);
                    // the first P.V of an item overwrites O_h: the previous item's epilogue must have read it
                    if (ok && u == 0 && na > 0) ok = mbar_wait(smem_u32(&sm.bar_o_empty[h]), (na - 1) & 1, abort_flag, p.status, kErrOEmpty);
                } else {
                    ok = mbar_wait(smem_u32(&sm.bar_kv_full[s]), (gs / kStages) & 1, abort_flag, p.status, kErrKFull);
                }
                if (ok && more) ok = mbar_wait(smem_u32(&sm.bar_kv_full[(gs + 2) % kStages]), ((gs + 2) / kStages) & 1, abort_flag, p.status, kErrKFull);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    if (active) {
                        issue_pv(s, buf, u == 0);
                        tc_commit(smem_u32(&sm.bar_pv_done[h]));
                        if (u == n2 - 1) tc_commit(smem_u32(&sm.bar_o_full[h]));
                    }
                    tc_commit(smem_u32(&sm.bar_kv_empty[s]));
                    if (more) {
                        if (active) {
                            issue_qk((gs + 2) % kStages, buf);
                            tc_commit(smem_u32(&sm.bar_s_full[h][buf]));
                        }
                        if (u + 3 == n2) tc_commit(smem_u32(&sm.bar_q_empty));      // that was the last Q.K^T of the item
                    }
                }
                __syncwarp();
            }
            g += n2;
            if (active) { gu += n2; ++na; }
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
    } else if (warp >= 4) {
        // =============================== softmax + epilogue ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsHigh));
        const int h = (warp - 4) / 4;                    // head slot
        const int row = (warp & 3) * 32 + lane;          // query row inside the tile == TMEM lane
        const uint32_t lane_addr = ((uint32_t)((warp & 3) * 32)) << 16;
        const uint32_t tS = tmem + lane_addr + h * 256;
        const uint32_t tO = tmem + lane_addr + h * 256 + 128;
        const float scale = p.scale_log2;
        uint32_t gu = 0, na = 0;                         // sub-tiles / items of this head so far
        uint32_t rounds = 0;                             // sub-tiles done in two-head items (MUFU turn taking)
        bool ok = true;
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = mbar_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            if (h < hd.nslots) {
                const bool pingpong = kPingPong && hd.nslots == 2;
                const int n2 = 2 * hd.n_kept;
                const int qpos = p.q_off + hd.t * kTile + row;   // position of this thread's query row in the KV sequence
                const int32_t* lim = p.lim + (size_t)hd.bh * p.Nc;
                float m_ref = -INFINITY, l_sum = 0.f;
                for (int u = 0; u < n2; ++u, ++gu) {
                    const int entry = sm.list[slot][u >> 1];
                    const int buf = u & 1;
                    const int k0 = (entry & 0x7fff) * kTile + buf * kSub;   // first key column of this sub-tile
                    const bool partial = (entry & 0x8000) != 0;
                    // visibility bits of this row for the 64 columns of a sub-tile that is not fully visible
                    uint32_t bits[2] = {0xffffffffu, 0xffffffffu};
                    if (partial) {
                        // columns this row may see: the causal prefix (and nothing past N), minus every chunk whose row limit is below it
                        const int nvis = max(0, min(min(qpos - k0 + 1, p.Nkv - k0), kSub));
#pragma unroll
                        for (int w = 0; w < 2; ++w) bits[w] = range_mask(0, nvis, w);
                        const int c_first = k0 / p.C, c_last = min((k0 + kSub - 1) / p.C, p.Nc - 1);
#pragma unroll 1
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            if (qpos > lim[cc]) {
                                const int lo = max(cc * p.C - k0, 0), hi = min((cc + 1) * p.C - k0, kSub);
#pragma unroll
                                for (int w = 0; w < 2; ++w) bits[w] &= ~range_mask(lo, hi, w);
                            }
                        }
                    }
                    ok = mbar_wait(smem_u32(&sm.bar_s_full[h][buf]), (gu >> 1) & 1, abort_flag, p.status, kErrSFull);
                    if (!ok) break;
                    tc_fence_after();
                    // the score row of this thread in registers: two loads in flight, one wait
                    uint32_t sreg[kSub];
                    tmem_ld32(tS + buf * kSub, *reinterpret_cast<uint32_t(*)[32]>(&sreg[0]));
                    tmem_ld32(tS + buf * kSub + 32, *reinterpret_cast<uint32_t(*)[32]>(&sreg[32]));
                    tc_wait_ld();
                    if (partial) {
#pragma unroll
                        for (int i = 0; i < kSub; ++i)
                            if (!((bits[i >> 5] >> (i & 31)) & 1u)) sreg[i] = 0xff800000u;      // -inf: exp2 gives exactly 0
                    }
                    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < kSub; i += 4) {
                        mx0 = fmaxf(mx0, __uint_as_float(sreg[i]));
                        mx1 = fmaxf(mx1, __uint_as_float(sreg[i + 1]));
                        mx2 = fmaxf(mx2, __uint_as_float(sreg[i + 2]));
                        mx3 = fmaxf(mx3, __uint_as_float(sreg[i + 3]));
                    }
                    const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale;       // scale > 0
                    // online softmax with lazy rescaling: the reference maximum only moves when the row max grew by > threshold
                    float alpha = 1.f;
                    bool need = false;
                    if (mx > m_ref + kRescaleThreshold) {           // also true for the first visible sub-tile (m_ref = -inf)
                        if (m_ref != -INFINITY) {                   // a row without visible entries so far has O = 0, l = 0
                            alpha = ex2(m_ref - mx);
                            l_sum *= alpha;
                            need = true;
                        }
                        m_ref = mx;
                    }
                    if (u > 0 && __any_sync(0xffffffffu, need)) {
                        // O_h is rescaled in place; the P.V of the previous sub-tile has to be complete first
                        ok = mbar_wait(smem_u32(&sm.bar_pv_done[h]), (gu - 1) & 1, abort_flag, p.status, kErrPvDone);
                        if (!ok) break;
                        tc_fence_after();
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
                    // The warps of the two heads that sit on the same scheduler share its MUFU pipe: they take turns for the
                    // exponentials (slot 0 first), so each runs them at the full rate while the other does its loads and maxima.
                    if (pingpong && (h == 1 || rounds > 0)) {
                        ok = mbar_wait(smem_u32(&sm.bar_mufu[h][warp & 3]), (h == 1 ? rounds : rounds - 1) & 1, abort_flag, p.status, kErrMufu);
                        if (!ok) break;
                    }
                    // P = exp2(S * scale - m), row sum in fp32, P packed to bf16 over the first 32 columns of this score buffer
                    float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
                    for (int c = 0; c < kSub / 32; ++c) {
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = ex2(fmaf(__uint_as_float(sreg[c * 32 + i]), scale, m_neg));
                            const float p1 = ex2(fmaf(__uint_as_float(sreg[c * 32 + i + 1]), scale, m_neg));
                            ls0 += p0;
                            ls1 += p1;
                            pk[i / 2] = pack_bf16(p0, p1);
                        }
                        tmem_st16(tS + buf * kSub + c * 16, pk);
                    }
                    l_sum += ls0 + ls1;
                    if (pingpong) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&sm.bar_mufu[h ^ 1][warp & 3]));
                        ++rounds;
                    }
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();                                 // every lane's P is in TMEM and fenced
                    if (lane == 0) mbar_arrive(smem_u32(&sm.bar_p_full[h][buf]));
                }
                // epilogue: O / l -> bf16 -> global; O_h is handed back to the issuer as soon as it sits in registers
                if (ok) ok = mbar_wait(smem_u32(&sm.bar_o_full[h]), na & 1, abort_flag, p.status, kErrOFull);
                if (ok) {
                    tc_fence_after();
                    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
                    const int qi = hd.t * kTile + row;           // query row
                    __nv_bfloat16* orow = p.o + (((size_t)hd.b * p.Hq + hd.head0 + h) * p.N + qi) * D;
                    uint32_t oreg[D];
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) tmem_ld32(tO + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&oreg[c * 32]));
                    tc_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sm.bar_o_empty[h]));
                    if (p.lse != nullptr && qi < p.N)
                        p.lse[((size_t)hd.b * p.Hq + hd.head0 + h) * p.N + qi] = l_sum > 0.f ? m_ref + log2f(l_sum) : -INFINITY;
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

// [heads, N, D] bf16 viewed as a 3-D tensor (D innermost); box = 64 x box_rows x 1 with 128-byte swizzle; rows past N read zero
// 3-D map over [heads, rows, D] bf16; consecutive heads are head_stride_rows rows apart (>= rows: a cache buffer is
// longer than the part of it that is valid; rows behind `rows` read as zero).
static int make_map(CUtensorMap* map, const void* base, int heads, int N, int D, int box_rows, long long head_stride_rows = 0) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(NATS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if (head_stride_rows <= 0) head_stride_rows = N;
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)heads};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)head_stride_rows * D * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NATS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return NATS_OK;
}

struct PrefillWs { size_t lim, tmax, tmin, counter, total; };
// N = rows of the KV sequence
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

// Tensor maps, parameters and launch shared by the entry points.  N query rows at positions q_off .. q_off + N - 1 of a
// KV sequence of Nkv rows whose heads are kv_head_stride rows apart (0: contiguous).
static int run_prefill(const void* d_q, const void* d_k, const void* d_v, void* d_o, int B, int Hq, int Hkv, int N, int Nkv,
                       int q_off, long long kv_head_stride, int D, int C, float sm_scale, const int32_t* lim,
                       const int32_t* tmax, const int32_t* tmin, int32_t* counter, int32_t* d_status, cudaStream_t st,
                       float* d_lse = nullptr) {
    CUtensorMap mq, mk, mv;
    if (int rc = make_map(&mq, d_q, B * Hq, N, D, 128)) return rc;
    if (int rc = make_map(&mk, d_k, B * Hkv, Nkv, D, kSub, kv_head_stride)) return rc;
    if (int rc = make_map(&mv, d_v, B * Hkv, Nkv, D, kSub, kv_head_stride)) return rc;
    PrefillParams p;
    p.o = (__nv_bfloat16*)d_o; p.lse = d_lse; p.lim = lim; p.tile_max = tmax; p.tile_min = tmin; p.status = d_status;
    p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.Nkv = Nkv; p.q_off = q_off; p.C = C;
    p.Nc = cdiv(Nkv, C); p.Nt = cdiv(N, kTile); p.Ntk = cdiv(Nkv, kTile);
    p.nrep = Hq / Hkv; p.n_groups = (p.nrep + 1) / 2;
    p.work_counter = counter;
    const long long items = (long long)B * Hkv * p.n_groups * p.Nt;
    NATS_CHECK_ARG(items <= 0x7fffffffLL - 65536, "too many work items (%lld)", items);
    p.total_items = (int)items;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    if (D == 64) return launch_prefill<64>(mq, mk, mv, p, B, st);
    return launch_prefill<128>(mq, mk, mv, p, B, st);
}

}  // namespace nats

using namespace nats;

extern "C" __attribute__((visibility("default"))) size_t nats_b200_prefill_workspace_bytes(int B, int Hkv, int N, int C) {
    if (B <= 0 || Hkv <= 0 || N <= 0 || C <= 0) return 0;
    return prefill_ws(B, Hkv, N, C).total;
}

static int prefill_first_call(const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
                              int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale,
                              void* d_workspace, size_t workspace_bytes, int64_t* d_kept_tiles, int32_t* d_status,
                              void* stream, float* d_lse, int32_t* d_n_visible) {
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
    if (d_n_visible != nullptr)
        if (int rc = nats_b200_visible_counts(lim, B, Hq, Hkv, N, C, d_n_visible, stream)) return rc;
    return run_prefill(d_q, d_k, d_v, d_o, B, Hq, Hkv, N, N, 0, 0, D, C, sm_scale, lim, tmax, tmin,
                       (int32_t*)(ws + w.counter), d_status, (cudaStream_t)stream, d_lse);
}

extern "C" __attribute__((visibility("default"))) int nats_b200_prefill_fwd(const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
                                     int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale,
                                     void* d_workspace, size_t workspace_bytes, int64_t* d_kept_tiles, int32_t* d_status,
                                     void* stream) {
    return prefill_first_call(d_q, d_k, d_v, d_o, d_roles, B, Hq, Hkv, N, D, C, SW, sm_scale, d_workspace, workspace_bytes,
                              d_kept_tiles, d_status, stream, nullptr, nullptr);
}

extern "C" __attribute__((visibility("default"))) int nats_b200_prefill_fwd_stats(
    const void* d_q, const void* d_k, const void* d_v, void* d_o, const uint8_t* d_roles,
    int B, int Hq, int Hkv, int N, int D, int C, int SW, float sm_scale, void* d_workspace, size_t workspace_bytes,
    int64_t* d_kept_tiles, float* d_lse, int32_t* d_n_visible, int32_t* d_status, void* stream) {
    NATS_CHECK_ARG(d_lse != nullptr && d_n_visible != nullptr, "null pointer");
    return prefill_first_call(d_q, d_k, d_v, d_o, d_roles, B, Hq, Hkv, N, D, C, SW, sm_scale, d_workspace, workspace_bytes,
                              d_kept_tiles, d_status, stream, d_lse, d_n_visible);
}


extern "C" __attribute__((visibility("default"))) size_t nats_b200_prefill_past_workspace_bytes(int B, int Hkv, int n_kv, int C) {
    if (B <= 0 || Hkv <= 0 || n_kv <= 0 || C <= 0) return 0;
    return prefill_ws(B, Hkv, n_kv, C).total;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_prefill_past_fwd(
    const void* d_q, const void* d_cache_k, const void* d_cache_v, void* d_o, const uint8_t* d_roles_new,
    const uint8_t* d_valid, int valid_stride, const int64_t* d_size_global, const int64_t* d_size_local,
    int B, int Hq, int Hkv, int x_len, int D, int C, int SW, int cache_capacity, int t0, int fill, int tail,
    float sm_scale, void* d_workspace, size_t workspace_bytes, int64_t* d_kept_tiles, int32_t* d_status, void* stream) {
    NATS_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && x_len > 0 && Hq % Hkv == 0, "bad shape B=%d Hq=%d Hkv=%d x_len=%d", B, Hq, Hkv, x_len);
    NATS_CHECK_ARG(C > 0 && SW > 0 && SW % C == 0, "sliding window %d must be a positive multiple of the chunk size %d", SW, C);
    NATS_CHECK_ARG(d_q && d_cache_k && d_cache_v && d_o && d_roles_new && d_valid && d_size_global && d_size_local &&
                   d_workspace && d_status, "null pointer");
    NATS_CHECK_ARG(((uintptr_t)d_q | (uintptr_t)d_cache_k | (uintptr_t)d_cache_v | (uintptr_t)d_o | (uintptr_t)d_workspace) % 16 == 0,
                   "q, the cache, o and the workspace must be 16-byte aligned");
    NATS_CHECK_ARG(sm_scale > 0.f, "sm_scale must be positive");
    NATS_CHECK_ARG(t0 >= SW && t0 % C == 0 && fill >= 0 && fill < C, "tail offset %d must be a multiple of the chunk size >= the window, fill %d in [0, chunk)", t0, fill);
    NATS_CHECK_ARG(tail >= 0 && tail < SW && tail % C == 0, "ring tail %d must be a multiple of the chunk size inside the window", tail);
    if (D != 64 && D != 128) return fail(NATS_ERR_UNSUPPORTED, "prefill supports head_dim 64 and 128, got %d", D);
    const long long n_kv = (long long)t0 + fill + x_len;
    NATS_CHECK_ARG(n_kv <= cache_capacity, "the cache holds %d rows, %lld are needed (the new tokens must have been appended)", cache_capacity, n_kv);
    NATS_CHECK_ARG(n_kv <= (long long)kMaxTiles * kTile, "cache + new tokens = %lld rows exceed the prefill limit %d", n_kv, kMaxTiles * kTile);
    const PrefillWs w = prefill_ws(B, Hkv, (int)n_kv, C);
    if (workspace_bytes < w.total)
        return fail(NATS_ERR_WORKSPACE, "prefill workspace: %zu bytes given, %zu needed", workspace_bytes, w.total);
    uint8_t* ws = (uint8_t*)d_workspace;
    int32_t* lim = (int32_t*)(ws + w.lim);
    int32_t* tmax = (int32_t*)(ws + w.tmax);
    int32_t* tmin = (int32_t*)(ws + w.tmin);
    if (int rc = nats_b200_role_prep_past(d_roles_new, d_valid, d_size_global, d_size_local, B, Hkv, x_len, C, SW,
                                          valid_stride, t0, fill, tail, lim, tmax, tmin, d_kept_tiles, stream)) return rc;
    return run_prefill(d_q, d_cache_k, d_cache_v, d_o, B, Hq, Hkv, x_len, (int)n_kv, t0 + fill, cache_capacity, D, C, sm_scale,
                       lim, tmax, tmin, (int32_t*)(ws + w.counter), d_status, (cudaStream_t)stream);
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


