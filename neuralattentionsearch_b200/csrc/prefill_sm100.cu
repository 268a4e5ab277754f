// Role-masked chunked flash-attention prefill for sm_100a: TMA-fed tcgen05.mma with TMEM accumulators.
//
// A work item = one 128-row query tile x one kv-head x up to two query heads of that kv-head's group.  The two heads
// share every K/V tile that is loaded and keep the tensor pipe busy in turns: while the softmax warps of one head
// work on its 128 x 128 score tile S = Q.K^T in TMEM, the tensor core runs the other head's O += P.V and next Q.K^T.
// The kernel is persistent: one CTA per SM takes items from a global counter (heaviest query tiles first).
//
//   warp 0      TMA producer: K and V of every kept KV tile, item after item, through one ring of tile-sized slots
//   warp 3      scheduler: fetches the next item, builds its kept-tile bitmap while the current item runs, loads its Q tiles
//   warps 1,2   MMA issuers of head slot 0 / 1 (one elected lane each): S_h = Q_h.K^T (SS, N = 128), O_h += P_h.V (TS, P from TMEM)
//   warps 4-7   softmax of head slot 0: one thread per query row, the 128-entry score row read with tcgen05.ld, online
//   warps 8-11  softmax of head slot 1  softmax in registers, P written back over S as packed bf16
//
// Which KV tiles are visited comes from the role bitmap: a bitmap of kept tiles is built in shared memory from the
// per-tile max / min row limits (nats_b200_role_prep); tiles without a visible entry are never loaded.  Only tiles
// whose min limit does not cover the whole query tile (and the diagonal) pay for per-element masking.
//
// TMEM (512 columns), head slot h: S_h [256 h, 256 h + 128), O_h [256 h + 128, 256 h + 128 + D); P_h (bf16) aliases
// the first 64 columns of S_h.  Every mbarrier wait is bounded: on a time-out the CTA raises the caller's status
// word, drains and exits.
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
#ifndef NATS_WAIT_LIMIT_NS
#define NATS_WAIT_LIMIT_NS (400ull * 1000ull * 1000ull)
#endif
constexpr unsigned long long kWaitLimitNs = NATS_WAIT_LIMIT_NS;

enum : int { kErrQ = 1, kErrKvFull, kErrKvEmpty, kErrSFull, kErrPFull, kErrOFull, kErrList, kErrOEmpty, kErrSmemAlign, kErrPipeLock };

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
    int Hq, Hkv, N, Nkv, q_off, C, Nc, Nt, Ntk, nrep, n_groups;   // n_groups = ceil(nrep / heads per item)
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

// L2 eviction priority of a TMA load: K / V tiles are read again by the CTAs that work on neighbouring query tiles and
// should stay, Q tiles are read once
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
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

// The same with the descriptors given as (low word, shared high word): within one kernel only the start address and
// the leading byte offset (low word) differ between operands, so the issuing thread adds small constants to 32-bit
// registers instead of carrying 64-bit descriptors around.
template <int ACC>
__device__ __forceinline__ void mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(ACC) : "memory");
}
template <int ACC>
__device__ __forceinline__ void mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(ACC) : "memory");
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

// 32-byte store (one sector) to a 32-byte aligned global address
__device__ __forceinline__ void st32(void* p, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
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

// packed fp32 pairs: one instruction for two lanes of a multiply-add or add
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

#ifdef NATS_TRACE
// development builds only: cycle stamps of one softmax warp and one issuer of CTA 0, summed per phase
__device__ unsigned long long g_trace[64];
#define TR_DECL(n) unsigned long long tr_acc[n] = {}; unsigned long long tr_t = clock64(); const bool tr_on = blockIdx.x == 0 && lane == 0
#define TR_RESET() do { tr_t = clock64(); } while (0)
#define TR(i) do { const unsigned long long t_ = clock64(); tr_acc[i] += t_ - tr_t; tr_t = t_; } while (0)
#define TR_DUMP(base, n) do { if (tr_on) for (int i_ = 0; i_ < n; ++i_) g_trace[base + i_] = tr_acc[i_]; } while (0)
#else
#define TR_DECL(n)
#define TR_RESET()
#define TR(i)
#define TR_DUMP(base, n)
#endif

// ---- shared memory --------------------------------------------------------------------------------
struct ItemHeader {
    int valid;      // 0: no more work
    int t;          // query tile
    int b, bh;      // batch index, b * Hkv + kv-head
    int head0;      // query head of slot 0
    int nslots;     // 1 or 2 query heads in this item
    int n_kept;     // kept 128-column KV tiles
    int pad;
};

constexpr int kBitWords = kMaxTiles / 32;

// K/V ring: slots of one 128-row tile each, filled in the order K_0 V_0 K_1 V_1 ... of the kept tiles (all items in
// one sequence).  A K slot is free again when both heads' Q.K^T of that tile have completed, a V slot after both P.V.
template <int D>
struct PrefillSmem {
    static constexpr int kHeads = D <= 128 ? 2 : 1;      // query heads of an item (head_dim 256: O fills the TMEM of one head pair)
    static constexpr int kSlots = D == 256 ? 2 : D == 128 ? 5 : 8;
    static constexpr uint32_t kTileBytes = 128 * D * 2;
    uint8_t q[kHeads][kTileBytes];             // one Q tile per head slot; D/64 boxes of 16 KB each
    uint8_t ring[kSlots][kTileBytes];          // K or V tile; D/64 boxes of 16 KB each
    uint32_t keep[2][kBitWords];               // bit kt: KV tile kt of the item has a visible entry (double buffered)
    uint32_t part[2][kBitWords];               // bit kt: the tile needs element masking
    ItemHeader item[2];
    unsigned long long bar_q_full[2], bar_q_empty[2];          // per head slot: its Q tile has landed / its last Q.K^T of the item is done
    unsigned long long bar_full[kSlots], bar_empty[kSlots];
    unsigned long long bar_s_full[2], bar_p_full[2][2], bar_o_full[2], bar_o_empty[2];
    unsigned long long bar_list_full[2], bar_list_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int pipe_lock;                             // held by the issuer whose batch of MMAs is being queued
};
static_assert(sizeof(PrefillSmem<128>) <= 232448 && sizeof(PrefillSmem<256>) <= 232448, "shared memory of the widest kernels");

constexpr int kListConsumers = 1 + 2 + 8;     // producer, two issuers, one lane of each of the eight softmax warps

// Walks the set bits of an item's kept-tile bitmap in ascending order.
struct TileWalk {
    const uint32_t* keep;
    const uint32_t* part;
    int w;
    uint32_t cur, pcur;
    __device__ __forceinline__ void init(const uint32_t* k, const uint32_t* p) {
        keep = k; part = p; w = 0; cur = k[0]; pcur = p[0];
    }
    // next kept tile; the caller asks for no more tiles than the item has
    __device__ __forceinline__ int next(bool& partial) {
        while (cur == 0u) { ++w; cur = keep[w]; pcur = part[w]; }
        const int b = __ffs(cur) - 1;
        cur &= cur - 1u;
        partial = (pcur >> b) & 1u;
        return w * 32 + b;
    }
};

// A bounded wait whose outcome is the same for every lane of the warp (all 32 lanes call it): lanes may see a time-out
// or the CTA's abort flag at different polls, and what follows (.sync.aligned instructions, __syncwarp) needs the
// whole warp on one path.
template <int RELAX = 0>
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status, int code) {
    const bool ok = mbar_wait<RELAX>(bar, parity, abort_flag, status, code);
    return __all_sync(0xffffffffu, ok);
}

// The two issuers queue their MMAs in whole batches (the P.V of a tile and the Q.K^T of the next): the tensor pipe runs
// MMAs in the order they were queued, so batches that interleaved would finish together and keep the two heads in step --
// both in their softmax, then both waiting for the tensor pipe.  With whole batches one head's scores are ready a batch
// earlier than the other's, and from then on one head's softmax overlaps the other head's MMAs.
#ifndef NATS_LOCK_SLEEP_NS
#define NATS_LOCK_SLEEP_NS 0       // pause between attempts to take the lock (0: none; 40 ns and 100 ns were measured slower)
#endif
__device__ __forceinline__ bool pipe_acquire(int* lock, int lane, volatile int* abort_flag, int32_t* status) {
    int got = 1;
    if (lane == 0) {
        if (atomicCAS(lock, 0, 1) != 0) {
            const unsigned long long t0 = global_ns();
            got = 0;
#pragma unroll 1
            for (uint32_t it = 0;; ++it) {
                if (NATS_LOCK_SLEEP_NS > 0) __nanosleep(NATS_LOCK_SLEEP_NS);
                if (atomicCAS(lock, 0, 1) == 0) { got = 1; break; }
                if ((it & 63u) == 63u) {
                    if (*abort_flag) break;
                    if (global_ns() - t0 > kWaitLimitNs) {
                        *abort_flag = 1;
                        atomicCAS(status, 0, kErrPipeLock);
                        break;
                    }
                }
            }
        }
    }
    return __shfl_sync(0xffffffffu, got, 0) != 0;
}
__device__ __forceinline__ void pipe_release(int* lock, int lane) {
    __syncwarp();
    if (lane == 0) atomicExch(lock, 0);
}

// Persistent kernel: every CTA takes work items (query tile x kv-head x head pair) from a global counter until none is
// left.  Per-item set-up (kept-tile bitmap, Q load) and tear-down (O -> global) overlap the main loops of the
// neighbouring items: warp 3 prepares the bitmap of the next item while the current one runs, the producer streams the
// next item's K/V through the same ring without a bubble, Q of the next item is loaded as soon as the last Q.K^T of the
// current one has completed, and a head's epilogue only delays that head's own chain.
//
// Per head and kept tile j the chain is  S = Q.K_j^T (8 or 4 MMAs of N = 128)  ->  softmax over the 128-entry row held in
// registers  ->  P (bf16) over the first 64 columns of S, handed over once per tile (a hand-over per half of 64 keys costs
// the softmax warps a second wait + fence + arrive and buys nothing, because a batch is queued whole: 1.16 against 1.13 ms)
// ->  O += P.V_j  ->  S = Q.K_{j+1}^T.  The two heads
// run this chain half a period apart, so that one head's softmax (MUFU and issue slots of the four SM sub-partitions)
// overlaps the other head's MMAs on the tensor pipe.
template <int D>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    using Smem = PrefillSmem<D>;
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    constexpr int NBOX = D / 64;                       // TMA boxes per tile
    constexpr int NS = Smem::kSlots;
    constexpr uint32_t TILE_BYTES = Smem::kTileBytes;  // one Q, K or V tile (128 rows)
    constexpr uint32_t IDESC_QK = instr_desc(kTile, false);
    constexpr uint32_t IDESC_PV = instr_desc(D, true);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    volatile int* abort_flag = &sm.abort_flag;

    if (tid == 0) {
        int bad = (*reinterpret_cast<volatile int32_t*>(p.status) != 0);
        if ((smem_u32(smem_raw) & 1023u) != 0u) {      // the swizzled tiles need a 1024-byte aligned base
            atomicCAS(p.status, 0, kErrSmemAlign);
            bad = 1;
        }
        sm.abort_flag = bad;
        sm.pipe_lock = 0;
    }
    __syncthreads();
    if (sm.abort_flag) return;                         // an earlier CTA gave up: do not start (uniform for the CTA)

    // ---- set-up: barriers, TMEM ----
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&sm.bar_full[s]), 1);
            mbar_init(smem_u32(&sm.bar_empty[s]), 2);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(smem_u32(&sm.bar_q_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_q_empty[h]), 1);              // one arrival per item and head slot
            mbar_init(smem_u32(&sm.bar_s_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_p_full[h][0]), 4);          // one arrival per softmax warp
            mbar_init(smem_u32(&sm.bar_p_full[h][1]), 4);
            mbar_init(smem_u32(&sm.bar_o_full[h]), 1);
            mbar_init(smem_u32(&sm.bar_o_empty[h]), 4);
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

    // Register budget: the softmax warpgroups get more registers (setmaxnreg.inc at the top of their branch), the
    // producer / issuer / scheduler warpgroup needs little and gives registers back.
    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLow));      // one site for the whole warpgroup

    if (warp == 3) {
        // =============================== scheduler: next work item and its kept-tile bitmap ===============================
        const int per_z = p.Nt * p.Hkv * p.n_groups;
        bool ok = true;
        int q_loads[2] = {0, 0};
        const uint64_t pol_q = l2_policy_evict_first();
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1, use = ic >> 1;
            if (use > 0) ok = warp_wait<kRelaxNs>(smem_u32(&sm.bar_list_empty[slot]), (use - 1) & 1, abort_flag, p.status, kErrList);
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
                for (int s0 = 0; s0 <= kt_last; s0 += 32) {        // tiles 0..kt_last with a visible entry
                    const int kt = s0 + lane;
                    const bool keep = kt <= kt_last && tmax[kt] >= q_lo;
                    // element masking is needed where the causal edge or a chunk's row limit cuts through the tile
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
                    hd.valid = 1; hd.t = t; hd.b = z; hd.bh = bh; hd.head0 = hkv * p.nrep + grp * Smem::kHeads;
                    hd.nslots = min(Smem::kHeads, p.nrep - grp * Smem::kHeads); hd.n_kept = n_kept; hd.pad = 0;
                    sm.item[slot] = hd;
                }
            } else if (lane == 0) {
                sm.item[slot].valid = 0;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.bar_list_full[slot]));
            if (!have) break;
            // Q of this item, head slot by head slot: a slot is reloaded as soon as that head's last Q.K^T of the previous
            // item has completed (the K/V producer is not held up by it, and one head does not wait for the other)
            const ItemHeader hd = sm.item[slot];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (!ok) break;
                if (ic > 0) ok = warp_wait<kRelaxNs>(smem_u32(&sm.bar_q_empty[h]), (ic - 1) & 1, abort_flag, p.status, kErrQ);
                if (!ok) break;
                if (h < hd.nslots) {
                    if (lane == 0) {
                        mbar_expect_tx(smem_u32(&sm.bar_q_full[h]), TILE_BYTES);
                        for (int x = 0; x < NBOX; ++x)
                            tma_load_3d(smem_u32(&sm.q[h][x * kBoxBytes]), &map_q, smem_u32(&sm.bar_q_full[h]), x * 64, hd.t * kTile,
                                        hd.b * p.Hq + hd.head0 + h, pol_q);
                    }
                    ++q_loads[h];
                }
                __syncwarp();
            }
        }
        if (!ok) {
            // given up: let Q copies that are still in flight land before the shared memory is released
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (q_loads[h] > 0) mbar_wait(smem_u32(&sm.bar_q_full[h]), (q_loads[h] - 1) & 1, nullptr, p.status, kErrQ);
        }
    } else if (warp == 0) {
        // =============================== TMA producer ===============================
        uint32_t g = 0;                                 // ring slots filled so far (all items): two per kept tile
        const uint64_t pol_kv = l2_policy_evict_last();
#ifdef NATS_TRACE
        unsigned long long tr_prod_wait = 0, tr_prod_n = 0;
        const unsigned long long tr_prod_t0 = clock64();
#endif
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
#ifdef NATS_TRACE
                    const unsigned long long tp0 = clock64();
#endif
                    if (g >= (uint32_t)NS) ok = warp_wait<kRelaxProdNs>(smem_u32(&sm.bar_empty[s]), ((g / NS) & 1) ^ 1, abort_flag, p.status, kErrKvEmpty);
#ifdef NATS_TRACE
                    tr_prod_wait += clock64() - tp0;
                    ++tr_prod_n;
#endif
                    if (!ok) break;
#ifdef NATS_TEST_WITHHOLD_FIRST_V
                    // test builds only: the V tile of a CTA's first kept tile is never loaded, so that a bounded wait runs out
                    const bool withhold = g == 1;
#else
                    const bool withhold = false;
#endif
                    if (lane == 0 && !withhold) {
                        mbar_expect_tx(smem_u32(&sm.bar_full[s]), TILE_BYTES);
                        const CUtensorMap* map = kv == 0 ? &map_k : &map_v;
                        for (int x = 0; x < NBOX; ++x)
                            tma_load_3d(smem_u32(&sm.ring[s][x * kBoxBytes]), map, smem_u32(&sm.bar_full[s]), x * 64, row0, hd.bh, pol_kv);
                    }
                    __syncwarp();
                }
            }
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
#ifdef NATS_TRACE
        if (blockIdx.x == 0 && lane == 0) { g_trace[32] = tr_prod_wait; g_trace[33] = tr_prod_n; g_trace[34] = clock64() - tr_prod_t0; }
#endif
        if (!ok) {
            // given up: let copies that are still in flight land before the shared memory is released
            for (uint32_t x = g > (uint32_t)NS ? g - NS : 0; x < g; ++x)
                mbar_wait(smem_u32(&sm.bar_full[x % NS]), (x / NS) & 1, nullptr, p.status, kErrKvFull);
        }
    } else if (warp == 1 || warp == 2) {
        // =============================== MMA issuers: warp 1 for head slot 0, warp 2 for head slot 1 ===============================
        // Per head and kept tile j:  O_h += P_j.V_j, then S_h = Q_h.K_{j+1}^T,
        // which overwrites P_j: the tensor pipe runs one thread's MMAs in issue order.  A ring slot is released when both
        // issuers have committed the MMAs that read it; an issuer whose head slot is empty in an item (odd group size)
        // only keeps the barrier counts going.
        const int h = warp - 1;
        constexpr uint32_t T16 = TILE_BYTES >> 4;
        // descriptors as (low word, high word): the high word (stride byte offset 1024, version, 128-byte swizzle) is the
        // same for Q, K and V; the low word holds the start address >> 4 and the leading byte offset >> 4
        const uint64_t q_desc = smem_desc(smem_u32(&sm.q[0][0]), 16, 1024) + (uint64_t)(h < Smem::kHeads ? h * T16 : 0);
        const uint64_t k_desc0 = smem_desc(smem_u32(&sm.ring[0][0]), 16, 1024);
        const uint64_t v_desc0 = smem_desc(smem_u32(&sm.ring[0][0]), kBoxBytes, 1024);
        const uint32_t desc_hi = (uint32_t)(q_desc >> 32);
        const uint32_t q_lo = (uint32_t)q_desc, k_lo0 = (uint32_t)k_desc0, v_lo0 = (uint32_t)v_desc0;
        const uint32_t tS = tmem + h * 256, tO = tmem + h * 256 + 128;
        auto issue_qk = [&](int s) {
            // S[128 x 128] = Q_h[128 x D] . K_j[128 x D]^T : D/16 MMAs of K = 16
            const uint32_t kl = k_lo0 + (uint32_t)s * T16;
            mma_ss_lo<0>(tS, q_lo, kl, desc_hi, IDESC_QK);
#pragma unroll
            for (int ks = 1; ks < D / 16; ++ks) {
                const uint32_t off = ((ks / 4) * kBoxBytes + (ks % 4) * 32) >> 4;
                mma_ss_lo<1>(tS, q_lo + off, kl + off, desc_hi, IDESC_QK);
            }
        };
        auto issue_pv_half = [&](int s, int half, bool first) {
            // O_h[128 x D] (+)= P_j[128 x 64 keys of this half] . V_j[64 x D] : 4 MMAs of K = 16; V is MN-major (D contiguous)
            const uint32_t vl = v_lo0 + (uint32_t)s * T16 + (uint32_t)(half * 4 * (2048 >> 4));
            const uint32_t aP = tS + half * 32;
            if (first) mma_ts_lo<0>(tO, aP, vl, desc_hi, IDESC_PV);
            else mma_ts_lo<1>(tO, aP, vl, desc_hi, IDESC_PV);
#pragma unroll
            for (int k4 = 1; k4 < 4; ++k4) mma_ts_lo<1>(tO, aP + k4 * 8, vl + (uint32_t)(k4 * (2048 >> 4)), desc_hi, IDESC_PV);
        };
        TR_DECL(8);
#ifdef NATS_TRACE
        unsigned long long tr_lock = 0, tr_pv = 0;
#endif
        uint32_t g = 0;          // ring slots consumed so far (all items, both issuers count alike)
        uint32_t gt = 0;         // tiles of this head (items in which its slot is used)
        uint32_t na = 0;         // items in which this head's slot was used
        bool ok = true;
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = warp_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            const int n = hd.n_kept;
            const bool active = h < hd.nslots;
            if (active) ok = warp_wait(smem_u32(&sm.bar_q_full[h]), na & 1, abort_flag, p.status, kErrQ);
            // ---- S of the first tile ----
            if (ok) ok = warp_wait(smem_u32(&sm.bar_full[g % NS]), (g / NS) & 1, abort_flag, p.status, kErrKvFull);
            if (ok && active) ok = pipe_acquire(&sm.pipe_lock, lane, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                if (active) {
                    issue_qk(g % NS);
                    tc_commit(smem_u32(&sm.bar_s_full[h]));
                } else {
                    // an empty head slot only keeps the counts going; for a used one the head's softmax warps release the
                    // ring slots and the Q tile when they see the scores (a commit costs the issuer ~50 cycles each)
                    mbar_arrive(smem_u32(&sm.bar_empty[g % NS]));
                    if (n == 1) mbar_arrive(smem_u32(&sm.bar_q_empty[h]));
                }
            }
            if (active) pipe_release(&sm.pipe_lock, lane);
            __syncwarp();
            // ---- tiles ----
            for (int j = 0; j < n && ok; ++j) {
                const uint32_t gv = g + 2 * j + 1;             // ring index of V_j; K_{j+1} follows it
                const int sv = gv % NS;
                TR(0);
                ok = warp_wait(smem_u32(&sm.bar_full[sv]), (gv / NS) & 1, abort_flag, p.status, kErrKvFull);
                TR(1);
                const bool more = j + 1 < n;
                const uint32_t gk = gv + 1;
                if (ok && active) {
                    TR(2);
                    // the first P.V of an item overwrites O_h: the previous item's epilogue must have read it
                    if (ok && j == 0 && na > 0) ok = warp_wait(smem_u32(&sm.bar_o_empty[h]), (na - 1) & 1, abort_flag, p.status, kErrOEmpty);
                    TR(3);
                    if (ok) ok = warp_wait(smem_u32(&sm.bar_p_full[h][1]), (gt + j) & 1, abort_flag, p.status, kErrPFull);
                    TR(4);
                }
                if (ok && more) ok = warp_wait(smem_u32(&sm.bar_full[gk % NS]), (gk / NS) & 1, abort_flag, p.status, kErrKvFull);
                TR(5);
                // everything the batch needs is there: queue it as a whole.  (The lock is never held across a wait for a
                // ring slot: the slot may be one the other head still has to release, which it can only do by queueing its
                // own batch.)
                if (ok && active) ok = pipe_acquire(&sm.pipe_lock, lane, abort_flag, p.status);
                if (!ok) break;
#ifdef NATS_TRACE
                { const unsigned long long t_ = clock64(); tr_lock += t_ - tr_t; tr_t = t_; }
#endif
                tc_fence_after();
                if (lane == 0) {
                    if (active) {
                        issue_pv_half(sv, 0, j == 0);
                        issue_pv_half(sv, 1, false);
                        if (!more) tc_commit(smem_u32(&sm.bar_o_full[h]));
                        tc_commit(smem_u32(&sm.bar_empty[sv]));        // V_j is free as soon as P.V has run: the ring is short
                    } else {
                        mbar_arrive(smem_u32(&sm.bar_empty[sv]));
                    }
#ifdef NATS_TRACE
                    { const unsigned long long t_ = clock64(); tr_pv += t_ - tr_t; tr_t = t_; }
#endif
                }
                if (lane == 0) {
                    if (more) {
                        if (active) {
                            issue_qk(gk % NS);
                            tc_commit(smem_u32(&sm.bar_s_full[h]));
                        } else {
                            mbar_arrive(smem_u32(&sm.bar_empty[gk % NS]));
                            if (j + 2 == n) mbar_arrive(smem_u32(&sm.bar_q_empty[h]));   // the last Q.K^T of the item
                        }
                    }
                }
                if (active) pipe_release(&sm.pipe_lock, lane);
                __syncwarp();
                TR(6);
#ifdef NATS_TRACE
                tr_acc[7] += 1;
#endif
            }
            g += 2 * n;
            if (active) { gt += n; ++na; }
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
#ifdef NATS_TRACE
        if (h == 0) { TR_DUMP(16, 8); if (tr_on) { g_trace[24] = tr_lock; g_trace[25] = tr_pv; } }
#endif
    } else if (warp >= 4) {
        // =============================== softmax + epilogue ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsHigh));
        const int h = (warp - 4) / 4;                    // head slot
        const int row = (warp & 3) * 32 + lane;          // query row inside the tile == TMEM lane
        const uint32_t lane_addr = ((uint32_t)((warp & 3) * 32)) << 16;
        const uint32_t tS = tmem + lane_addr + h * 256;
        const uint32_t tO = tmem + lane_addr + h * 256 + 128;
        const float scale = p.scale_log2;
        const bool o_wide = (reinterpret_cast<uintptr_t>(p.o) & 31u) == 0;     // 32-byte stores need a 32-byte aligned output
        uint32_t gt = 0, na = 0;                         // tiles / items of this head so far
        uint32_t g = 0;                                  // ring slots of all items so far (two per kept tile), as the issuers count
        const bool releaser = (warp & 3) == 0 && lane == 0;   // one thread per head frees ring slots and the Q tile
        bool ok = true;
        TR_DECL(10);
#ifdef NATS_TRACE
        unsigned long long tr_epi_ld = 0;
#endif
        for (int ic = 0; ok; ++ic) {
            const int slot = ic & 1;
            ok = warp_wait(smem_u32(&sm.bar_list_full[slot]), (ic >> 1) & 1, abort_flag, p.status, kErrList);
            if (!ok) break;
            const ItemHeader hd = sm.item[slot];
            if (!hd.valid) break;
            TR(8);
            if (h < hd.nslots) {
                const int n = hd.n_kept;
                const int qpos = p.q_off + hd.t * kTile + row;   // position of this thread's query row in the KV sequence
                const int32_t* lim = p.lim + (size_t)hd.bh * p.Nc;
                float m_ref = -INFINITY, l_sum = 0.f;
                TileWalk walk;
                walk.init(sm.keep[slot], sm.part[slot]);
                for (int j = 0; j < n; ++j, ++gt) {
                    bool partial;
                    const int k0 = walk.next(partial) * kTile;    // first key column of this tile
                    // visibility bits of this row for the 128 columns of a tile that is not fully visible
                    uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
                    if (partial) {
                        // columns this row may see: the causal prefix (and nothing past Nkv), minus every chunk whose row limit is below it
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
                    // S of tile j is complete; so is O += P.V of tile j - 1, which the same thread issued in front of it
                    TR(0);
                    ok = warp_wait(smem_u32(&sm.bar_s_full[h]), gt & 1, abort_flag, p.status, kErrSFull);
                    if (!ok) break;
                    tc_fence_after();
                    if (releaser) {
                        // Q.K^T of tile j is complete: this head is done with K_j and, on the item's last tile, with its Q tile
                        mbar_arrive(smem_u32(&sm.bar_empty[(g + 2 * j) % NS]));
                        if (j == n - 1) mbar_arrive(smem_u32(&sm.bar_q_empty[h]));
                    }
                    TR(1);
                    // the score row of this thread in registers: four loads in flight, one wait
                    uint32_t sreg[kTile];
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sreg[c * 32]));
                    tc_wait_ld();
                    TR(2);
                    if (partial) {
#pragma unroll
                        for (int i = 0; i < kTile; ++i)
                            if (!((bits[i >> 5] >> (i & 31)) & 1u)) sreg[i] = 0xff800000u;      // -inf: exp2 gives exactly 0
                    }
                    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < kTile; i += 8) {
                        mx0 = max3(mx0, __uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1]));
                        mx1 = max3(mx1, __uint_as_float(sreg[i + 2]), __uint_as_float(sreg[i + 3]));
                        mx2 = max3(mx2, __uint_as_float(sreg[i + 4]), __uint_as_float(sreg[i + 5]));
                        mx3 = max3(mx3, __uint_as_float(sreg[i + 6]), __uint_as_float(sreg[i + 7]));
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
                    if (j > 0 && __any_sync(0xffffffffu, need)) {
                        // O_h is rescaled in place (the P.V of the previous tile is complete, see above)
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
                    // P = exp2(S * scale - m), row sum in fp32, P packed to bf16 over the first 64 columns of S
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
                        // a batch is queued when all of P is there: one hand-over per tile (wait, fence, arrive), not one per half
                        if (half == 1) {
                            tc_wait_st();
                            tc_fence_before();
                            __syncwarp();                         // every lane's row of P is in TMEM and fenced
                            if (lane == 0) mbar_arrive(smem_u32(&sm.bar_p_full[h][1]));
                        }
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
                // epilogue: O / l -> bf16 -> global; O_h is handed back to the issuer as soon as it sits in registers
                TR(0);
                if (ok) ok = warp_wait(smem_u32(&sm.bar_o_full[h]), na & 1, abort_flag, p.status, kErrOFull);
                TR(6);
                if (ok) {
                    tc_fence_after();
                    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
                    const int qi = hd.t * kTile + row;           // query row
                    __nv_bfloat16* orow = p.o + (((size_t)hd.b * p.Hq + hd.head0 + h) * p.N + qi) * D;
                    constexpr int OW = D < 128 ? D : 128;          // columns of O held in registers at a time
                    if (p.lse != nullptr && qi < p.N)
                        p.lse[((size_t)hd.b * p.Hq + hd.head0 + h) * p.N + qi] = l_sum > 0.f ? m_ref + log2f(l_sum) : -INFINITY;
#pragma unroll 1
                    for (int c0 = 0; c0 < D; c0 += OW) {
                        uint32_t oreg[OW];
#pragma unroll
                        for (int c = 0; c < OW / 32; ++c) tmem_ld32(tO + c0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&oreg[c * 32]));
                        tc_wait_ld();
                        if (c0 + OW >= D) {                          // O_h is in registers: hand it back to the issuer
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&sm.bar_o_empty[h]));
                        }
#ifdef NATS_TRACE
                        { const unsigned long long t_ = clock64(); tr_epi_ld += t_ - tr_t; tr_t = t_; }
#endif
                        if (qi < p.N) {
                            // a thread owns a whole output row (D * 2 bytes): 32-byte stores, one full sector each
#pragma unroll
                            for (int i = 0; i < OW; i += 16) {
                                uint32_t w[8];
#pragma unroll
                                for (int x = 0; x < 8; ++x)
                                    w[x] = pack_bf16(__uint_as_float(oreg[i + 2 * x]) * inv, __uint_as_float(oreg[i + 2 * x + 1]) * inv);
                                if (o_wide) {
                                    st32(orow + c0 + i, w);
                                } else {
                                    st16(orow + c0 + i, make_uint4(w[0], w[1], w[2], w[3]));
                                    st16(orow + c0 + i + 8, make_uint4(w[4], w[5], w[6], w[7]));
                                }
                            }
                        }
                    }
                }
                ++na;
                TR(7);
#ifdef NATS_TRACE
                tr_acc[9] += n;
#endif
            }
            g += 2 * hd.n_kept;
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(smem_u32(&sm.bar_list_empty[slot]));
        }
#ifdef NATS_TRACE
        if (warp == 4) { TR_DUMP(0, 10); if (tr_on) g_trace[10] = tr_epi_ld; }
#endif
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

}  // namespace nats

#include "prefill_pair.cuh"

namespace nats {

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

constexpr int kMaxDevices = 64;

template <int D>
static int launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p,
                          cudaStream_t st) {
    const size_t smem = sizeof(PrefillSmem<D>);
    int dev = 0, sms = 0;
    NATS_CHECK_CUDA(cudaGetDevice(&dev));
    // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel
    static bool attr_set[kMaxDevices] = {};
    if (dev < 0 || dev >= kMaxDevices || !attr_set[dev]) {
        NATS_CHECK_CUDA(cudaFuncSetAttribute(prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < kMaxDevices) attr_set[dev] = true;
    }
    NATS_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    NATS_CHECK_CUDA(cudaMemsetAsync(p.work_counter, 0, sizeof(int32_t), st));
    const int grid = p.total_items < sms ? p.total_items : sms;      // one persistent CTA per SM
    prefill_kernel<D><<<grid, kPrefillThreads, smem, st>>>(mq, mk, mv, p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

static int launch_prefill_pair(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, cudaStream_t st) {
    const size_t smem = sizeof(PairSmem);
    int dev = 0, sms = 0;
    NATS_CHECK_CUDA(cudaGetDevice(&dev));
    static bool attr_set[kMaxDevices] = {};
    if (dev < 0 || dev >= kMaxDevices || !attr_set[dev]) {
        NATS_CHECK_CUDA(cudaFuncSetAttribute(prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < kMaxDevices) attr_set[dev] = true;
    }
    NATS_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int grid = 2 * p.total_items < sms ? 2 * p.total_items : sms;        // one persistent CTA pair per SM pair
    grid &= ~1;
    prefill_pair_kernel<<<grid, kPrefillThreads, smem, st>>>(mq, mk, mv, p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

// CTA pairs (cta_group::2) for head_dim 128 and group sizes that are a multiple of four; NATS_B200_PAIR=0 turns them off
static bool use_pair_kernel(int D, int nrep) {
    static int mode = -1;
    if (mode < 0) {
        const char* e = getenv("NATS_B200_PAIR");
        mode = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return mode == 1 && D == 128 && nrep % 4 == 0;
}

// Tensor maps, parameters and launch shared by the entry points.  N query rows at positions q_off .. q_off + N - 1 of a
// KV sequence of Nkv rows whose heads are kv_head_stride rows apart (0: contiguous).
static int run_prefill(const void* d_q, const void* d_k, const void* d_v, void* d_o, int B, int Hq, int Hkv, int N, int Nkv,
                       int q_off, long long kv_head_stride, int D, int C, float sm_scale, const int32_t* lim,
                       const int32_t* tmax, const int32_t* tmin, int32_t* counter, int32_t* d_status, cudaStream_t st,
                       float* d_lse = nullptr) {
    const bool pair = use_pair_kernel(D, Hq / Hkv);
    CUtensorMap mq, mk, mv;
    if (int rc = make_map(&mq, d_q, B * Hq, N, D, 128)) return rc;
    if (int rc = make_map(&mk, d_k, B * Hkv, Nkv, D, pair ? 64 : 128, kv_head_stride)) return rc;     // a pair's CTA loads half the rows of a K tile
    if (int rc = make_map(&mv, d_v, B * Hkv, Nkv, D, 128, kv_head_stride)) return rc;
    PrefillParams p;
    p.o = (__nv_bfloat16*)d_o; p.lse = d_lse; p.lim = lim; p.tile_max = tmax; p.tile_min = tmin; p.status = d_status;
    p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.Nkv = Nkv; p.q_off = q_off; p.C = C;
    p.Nc = cdiv(Nkv, C); p.Nt = cdiv(N, kTile); p.Ntk = cdiv(Nkv, kTile);
    const int heads_per_item = D <= 128 ? 2 : 1;
    p.nrep = Hq / Hkv; p.n_groups = (p.nrep + heads_per_item - 1) / heads_per_item;
    p.work_counter = counter;
    const long long items = (long long)B * Hkv * p.n_groups * p.Nt;
    NATS_CHECK_ARG(items <= 0x7fffffffLL - 65536, "too many work items (%lld)", items);
    p.total_items = (int)items;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    if (pair) {
        p.n_groups = p.nrep / 4;
        p.total_items = B * Hkv * p.n_groups * p.Nt;
        return launch_prefill_pair(mq, mk, mv, p, st);
    }
    if (D == 64) return launch_prefill<64>(mq, mk, mv, p, st);
    if (D == 256) return launch_prefill<256>(mq, mk, mv, p, st);
    return launch_prefill<128>(mq, mk, mv, p, st);
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
    if (D != 64 && D != 128 && D != 256) return fail(NATS_ERR_UNSUPPORTED, "prefill supports head_dim 64, 128 and 256, got %d", D);
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
    if (D != 64 && D != 128 && D != 256) return fail(NATS_ERR_UNSUPPORTED, "prefill supports head_dim 64, 128 and 256, got %d", D);
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



#ifdef NATS_TRACE
extern "C" __attribute__((visibility("default"))) int nats_b200_debug_trace(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, nats::g_trace, sizeof(unsigned long long) * 64) == cudaSuccess ? 0 : 1;
}
#endif
