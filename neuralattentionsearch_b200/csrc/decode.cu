// Decode attention over the compacted ragged cache: split-KV, GQA-aware, HBM-bound.
//
// One block owns kSeg consecutive tokens of the *logical* sequence of one (batch, kv-head):
//     [ valid ring slots | kept tokens [SW,len) | tokens of the unfinished chunk [T0,T0+fill) | the new token ]
// and its four warps take 16-token tiles of it in turn.  A tile's K and V rows travel global -> shared memory with
// cp.async (16 bytes per lane, bypassing L1) through a per-warp ring of kDecStages tiles, so two tiles are in flight
// while one is consumed and the bytes in flight cost no registers.  All query heads of the group are served by the one
// read: S = Q.K^T runs as mma.sync m16n8k16 with the (up to 8) query heads as the M rows and 8 tokens as N; the
// score fragments are exactly the A fragments of O += P.V, so P never leaves registers.  The instruction count per byte
// is then small enough that the kernel is limited by HBM, not by issue slots.
// Blocks of a (batch, kv-head) leave partial (max, sum, acc) in the workspace; the block that arrives last combines
// them (an atomic ticket, nobody waits).  The block owning the last logical token also appends it to the cache.
#include "common.cuh"

namespace nats {

#ifndef NATS_DEC_SEG
#define NATS_DEC_SEG 1024
#endif
#ifndef NATS_DEC_STAGES
#define NATS_DEC_STAGES 3
#endif
constexpr int kSeg = NATS_DEC_SEG;          // logical tokens per block
constexpr int kDecStages = NATS_DEC_STAGES; // ring depth per warp
constexpr int kDecThreads = 128;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kTileTok = 16;                // tokens per warp tile
constexpr int kMaxRep = 8;                  // query heads per kv-head the fragment rows cover (rows 8..15 stay zero)

struct DecodeParams {
    const __nv_bfloat16* q;        // [B,Hq,1,D]
    const __nv_bfloat16* k_new;    // [B,Hkv,1,D]
    const __nv_bfloat16* v_new;
    __nv_bfloat16* o;              // [B,Hq,1,D]
    __nv_bfloat16* ck;             // [B,Hkv,Lcap,D]
    __nv_bfloat16* cv;
    uint8_t* valid;                // [B,Hkv,Lcap]
    const long long* size_global;  // [B,Hkv]
    const long long* size_local;
    const int32_t* state;          // [0] = T0
    int32_t* counters;             // [B*Hkv]   (workspace)
    float* partials;               // [B*Hkv, max_splits, nrep, D+2]   (workspace)
    int Hq, Hkv, nrep, Lcap, SW, fill, max_splits;
    int fill_from_state;           // 1: the number of tokens in the unfinished chunk is read from state[4] (static launches)
    float scale_log2;              // sm_scale * log2(e)
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 16-byte asynchronous global -> shared copy that bypasses L1; with valid == false nothing is read and zeros are written
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D (16x8, fp32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <int D>
__global__ void __launch_bounds__(kDecThreads) decode_kernel(const DecodeParams p) {
    constexpr int ROWB = D * 2;                      // bytes of a K or V row
    constexpr int CHUNKS = ROWB / 16;                // 16-byte chunks per row: 16 (D = 128) or 8 (D = 64)
    constexpr int TILE_BYTES = kTileTok * ROWB;      // one tile of K (and as much again of V)
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    constexpr int CP_PER_LANE = kTileTok * CHUNKS / 32;   // cp.async per lane for one of K / V
    constexpr int ROWS_PER_CP = 32 / CHUNKS;         // rows one warp-wide cp.async covers
    constexpr unsigned FULL = 0xffffffffu;
    const float NEG_INF = -INFINITY;

    const int seg = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const int bh = b * p.Hkv + hkv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nrep = p.nrep;
    const int len = (int)(p.size_global[bh] + p.size_local[bh]);
    const int T0 = p.state[0];
    const int fill = p.fill_from_state ? p.state[4] : p.fill;
    const int Ltot = len + fill + 1;
    const int nsplit = (Ltot + kSeg - 1) / kSeg;
    if (seg >= nsplit) return;
    const int r0 = seg * kSeg, r1 = min(Ltot, r0 + kSeg);

    extern __shared__ __align__(128) uint8_t dsm[];
    __shared__ __align__(16) uint8_t s_ring_ok[kSeg];
    __shared__ int s_last;
    // after the main loop the ring memory holds the per-warp partial results
    float (*s_acc)[kMaxRep][D] = reinterpret_cast<float (*)[kMaxRep][D]>(dsm);
    float (*s_m)[kMaxRep] = reinterpret_cast<float (*)[kMaxRep]>(dsm + kDecWarps * kMaxRep * D * 4);
    float (*s_l)[kMaxRep] = reinterpret_cast<float (*)[kMaxRep]>(dsm + kDecWarps * kMaxRep * (D + 1) * 4);
    static_assert(kDecWarps * kMaxRep * (D + 2) * 4 <= kDecWarps * kDecStages * STAGE_BYTES, "combine scratch must fit into the ring");

    const __nv_bfloat16* ck = p.ck + (size_t)bh * p.Lcap * D;
    const __nv_bfloat16* cv = p.cv + (size_t)bh * p.Lcap * D;
    const uint8_t* valid = p.valid + (size_t)bh * p.Lcap;
    const __nv_bfloat16* kn = p.k_new + (size_t)bh * D;
    const __nv_bfloat16* vn = p.v_new + (size_t)bh * D;

    if (r0 < p.SW) {
        for (int i = tid; i < kSeg; i += kDecThreads) s_ring_ok[i] = (r0 + i < p.SW) ? valid[r0 + i] : 1;
    }
    // the block that owns the last logical token appends it (nobody reads that cache row in this launch)
    if (r1 == Ltot && warp == 0 && lane < CHUNKS) {
        const size_t dst = ((size_t)bh * p.Lcap + T0 + fill) * D + lane * 8;
        st16(p.ck + dst, ld16(kn + lane * 8));
        st16(p.cv + dst, ld16(vn + lane * 8));
        if (lane == 0) p.valid[(size_t)bh * p.Lcap + T0 + fill] = 1;
    }
    // Q as A fragments (rows = query heads of the group, 16 dims per k-step); rows >= nrep and rows 8..15 are zero
    const int hrow = lane >> 2, quad = lane & 3;
    uint32_t qa[D / 16][2];
    {
        const __nv_bfloat16* qrow = p.q + ((size_t)b * p.Hq + (size_t)hkv * nrep + hrow) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qa[ks][0] = hrow < nrep ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + quad * 2) : 0u;
            qa[ks][1] = hrow < nrep ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + quad * 2) : 0u;
        }
    }
    if (r0 < p.SW) __syncthreads();

    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dsm) + warp * kDecStages * STAGE_BYTES;
    const int n_tiles = (r1 - r0 + kTileTok - 1) / kTileTok;            // tiles of this block
    const int my_tiles = (n_tiles - warp + kDecWarps - 1) / kDecWarps;   // tiles warp, warp + 4, ... are this warp's

    // issue the copies of this warp's it-th tile: row r of the tile, chunk c goes to r*ROWB + ((c ^ (r & 7)) * 16)
    auto issue = [&](int it) {
        const int i0 = r0 + (it * kDecWarps + warp) * kTileTok;
        const uint32_t dst = ring + (it % kDecStages) * STAGE_BYTES;
        const int c = lane % CHUNKS, rsub = lane / CHUNKS;
        if (i0 + kTileTok <= p.SW) {
            // a ring tile none of whose slots is valid (a whole chunk that was not a sliding one) is not read at all
            const uint4 f = *reinterpret_cast<const uint4*>(&s_ring_ok[i0 - r0]);
            if ((f.x | f.y | f.z | f.w) == 0u) return;
        }
        if (i0 + kTileTok <= len) {                      // whole tile inside ring + kept tokens: logical == physical
            const __nv_bfloat16* kp = ck + (size_t)i0 * D + c * 8;
            const __nv_bfloat16* vp = cv + (size_t)i0 * D + c * 8;
#pragma unroll
            for (int x = 0; x < CP_PER_LANE; ++x) {
                const int r = x * ROWS_PER_CP + rsub;
                const uint32_t off = r * ROWB + ((c ^ (r & 7)) << 4);
                cp_async16(dst + off, kp + (size_t)r * D, true);
                cp_async16(dst + TILE_BYTES + off, vp + (size_t)r * D, true);
            }
        } else {
#pragma unroll
            for (int x = 0; x < CP_PER_LANE; ++x) {
                const int r = x * ROWS_PER_CP + rsub;
                const int i = i0 + r;
                const bool ok = i < r1;
                const __nv_bfloat16 *kp = ck, *vp = cv;
                if (ok) {
                    if (i < len) { kp = ck + (size_t)i * D; vp = cv + (size_t)i * D; }
                    else if (i < len + fill) { const size_t ph = (size_t)(T0 + (i - len)); kp = ck + ph * D; vp = cv + ph * D; }
                    else { kp = kn; vp = vn; }
                }
                const uint32_t off = r * ROWB + ((c ^ (r & 7)) << 4);
                cp_async16(dst + off, kp + c * 8, ok);
                cp_async16(dst + TILE_BYTES + off, vp + c * 8, ok);
            }
        }
    };

    float oacc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) { oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f; }
    float m_run = NEG_INF, l_run = 0.f;              // of query head `hrow`; l is this lane's share until the end

#pragma unroll
    for (int it = 0; it < kDecStages - 1; ++it) {
        if (it < my_tiles) issue(it);
        cp_async_commit();
    }
    for (int it = 0; it < my_tiles; ++it) {
        __syncwarp();                                // every lane is done reading the stage that is refilled now
        if (it + kDecStages - 1 < my_tiles) issue(it + kDecStages - 1);
        cp_async_commit();
        cp_async_wait<kDecStages - 1>();
        __syncwarp();                                // ... and sees the other lanes' copies of the stage consumed now
        const int i0 = r0 + (it * kDecWarps + warp) * kTileTok;
        const uint32_t sk = ring + (it % kDecStages) * STAGE_BYTES, sv = sk + TILE_BYTES;
        unsigned vmask = 0xffffu;                    // which of the 16 tokens exist and are valid
        if (i0 < p.SW || i0 + kTileTok > r1) {
            bool ok = false;
            if (lane < kTileTok) {
                const int i = i0 + lane;
                ok = i < r1 && (i >= p.SW || s_ring_ok[i - r0] != 0);
            }
            vmask = __ballot_sync(FULL, ok) & 0xffffu;
            if (vmask == 0u) continue;               // nothing visible in this tile (its copies were skipped as well)
        }
        // ---- S[heads x 16 tokens] = Q . K^T ----
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
            const int r = nt * 8 + (lane & 7);
#pragma unroll
            for (int kp = 0; kp < D / 32; ++kp) {
                uint32_t kb[4];
                const int chunk = kp * 4 + (lane >> 3);
                ldmatrix_x4(sk + r * ROWB + ((chunk ^ (r & 7)) << 4), kb);
                mma_bf16(sc[nt], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, kb[0], kb[1]);
                mma_bf16(sc[nt], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, kb[2], kb[3]);
            }
        }
        // ---- online softmax of head `hrow` over the 4 scores this lane holds (tokens nt*8 + quad*2 + {0,1}) ----
        float s[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int t = nt * 8 + quad * 2 + e;
                s[nt * 2 + e] = ((vmask >> t) & 1u) ? sc[nt][e] * p.scale_log2 : NEG_INF;
            }
        float mt = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
        mt = fmaxf(mt, __shfl_xor_sync(FULL, mt, 1));
        mt = fmaxf(mt, __shfl_xor_sync(FULL, mt, 2));
        const float m_new = fmaxf(m_run, mt);
        const float mu = (m_new == NEG_INF) ? 0.f : m_new;
        const float alpha = fast_exp2(m_run - mu);
        const float p0 = fast_exp2(s[0] - mu), p1 = fast_exp2(s[1] - mu), p2 = fast_exp2(s[2] - mu), p3 = fast_exp2(s[3] - mu);
        l_run = l_run * alpha + (p0 + p1) + (p2 + p3);
        m_run = m_new;
        if (__any_sync(FULL, alpha != 1.f)) {
#pragma unroll
            for (int n = 0; n < D / 8; ++n) { oacc[n][0] *= alpha; oacc[n][1] *= alpha; }
        }
        const uint32_t pa0 = pack2_bf16(p0, p1), pa2 = pack2_bf16(p2, p3);
        // ---- O[heads x D] += P . V ----
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
            uint32_t vb[4];
            const int r = ((lane >> 3) & 1) * 8 + (lane & 7);
            const int chunk = np * 2 + (lane >> 4);
            ldmatrix_x4_trans(sv + r * ROWB + ((chunk ^ (r & 7)) << 4), vb);
            mma_bf16(oacc[2 * np], pa0, 0u, pa2, 0u, vb[0], vb[1]);
            mma_bf16(oacc[2 * np + 1], pa0, 0u, pa2, 0u, vb[2], vb[3]);
        }
    }

    // ---- combine the warps of this block (the ring is drained first: its memory is reused) ----
    cp_async_wait<0>();
    __syncthreads();
    l_run += __shfl_xor_sync(FULL, l_run, 1);
    l_run += __shfl_xor_sync(FULL, l_run, 2);
    if (hrow < nrep) {
        if (quad == 0) { s_m[warp][hrow] = m_run; s_l[warp][hrow] = l_run; }
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<float2*>(&s_acc[warp][hrow][n * 8 + quad * 2]) = make_float2(oacc[n][0], oacc[n][1]);
    }
    __syncthreads();
    constexpr int PSTRIDE = D + 2;
    float* part_out = p.partials + ((size_t)bh * p.max_splits + seg) * nrep * PSTRIDE;
    for (int idx = tid; idx < nrep * D; idx += kDecThreads) {
        const int h = idx / D, d = idx % D;
        float mf = NEG_INF;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) mf = fmaxf(mf, s_m[w][h]);
        const float mu = (mf == NEG_INF) ? 0.f : mf;
        float a = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float wgt = fast_exp2(s_m[w][h] - mu);
            a = fmaf(s_acc[w][h][d], wgt, a);
            l = fmaf(s_l[w][h], wgt, l);
        }
        if (nsplit == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            p.o[((size_t)b * p.Hq + (size_t)hkv * nrep + h) * D + d] = __float2bfloat16_rn(a * inv);
        } else {
            part_out[h * PSTRIDE + d] = a;
            if (d == 0) { part_out[h * PSTRIDE + D] = mf; part_out[h * PSTRIDE + D + 1] = l; }
        }
    }
    if (nsplit == 1) return;
    // ---- the last block of this (batch, kv-head) combines the splits ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int ticket = atomicAdd(&p.counters[bh], 1);
        s_last = (ticket == nsplit - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* parts = p.partials + (size_t)bh * p.max_splits * nrep * PSTRIDE;
    for (int idx = tid; idx < nrep * D; idx += kDecThreads) {
        const int h = idx / D, d = idx % D;
        float mf = NEG_INF;
        for (int s = 0; s < nsplit; ++s) mf = fmaxf(mf, __ldcg(parts + ((size_t)s * nrep + h) * PSTRIDE + D));
        const float mu = (mf == NEG_INF) ? 0.f : mf;
        float a = 0.f, l = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float* ps = parts + ((size_t)s * nrep + h) * PSTRIDE;
            const float wgt = fast_exp2(__ldcg(ps + D) - mu);
            a = fmaf(__ldcg(ps + d), wgt, a);
            l = fmaf(__ldcg(ps + D + 1), wgt, l);
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        p.o[((size_t)b * p.Hq + (size_t)hkv * nrep + h) * D + d] = __float2bfloat16_rn(a * inv);
    }
    if (tid == 0) p.counters[bh] = 0;
}

template <int D>
static cudaError_t launch_decode(const DecodeParams& p, dim3 grid, cudaStream_t st) {
    constexpr int smem = kDecWarps * kDecStages * 2 * kTileTok * D * 2;
    // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel
    constexpr int kMaxDev = 64;
    static bool attr_set[kMaxDev] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDev || !attr_set[dev]) {
        e = cudaFuncSetAttribute(decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < kMaxDev) attr_set[dev] = true;
    }
    decode_kernel<D><<<grid, kDecThreads, smem, st>>>(p);
    return cudaGetLastError();
}

static size_t decode_counter_bytes(int B, int Hkv) { return align_up((size_t)B * Hkv * sizeof(int32_t), 256); }
static int decode_max_splits(int max_len) { return cdiv(max_len + 1, kSeg); }

}  // namespace nats

using namespace nats;

extern "C" __attribute__((visibility("default"))) size_t nats_b200_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_len) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || max_len < 0 || Hq % Hkv) return 0;
    const int nrep = Hq / Hkv;
    return decode_counter_bytes(B, Hkv) +
           (size_t)B * Hkv * decode_max_splits(max_len) * nrep * (D + 2) * sizeof(float);
}

static int decode_impl(const void* d_q, const void* d_k_new, const void* d_v_new, void* d_o,
                       void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                       const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                       int fill, int max_len_bound, int fill_from_state,
                       int B, int Hq, int Hkv, int D, int C, int SW, float sm_scale,
                       void* d_workspace, size_t workspace_bytes, void* stream) {
    NATS_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "bad head counts B=%d Hq=%d Hkv=%d", B, Hq, Hkv);
    NATS_CHECK_ARG(C > 0 && SW > 0 && SW % C == 0, "sliding window %d must be a positive multiple of the chunk size %d", SW, C);
    NATS_CHECK_ARG(d_q && d_k_new && d_v_new && d_o && d_cache_k && d_cache_v && d_valid && d_size_global && d_size_local &&
                   d_state && d_workspace, "null pointer");
    NATS_CHECK_ARG(((uintptr_t)d_q | (uintptr_t)d_k_new | (uintptr_t)d_v_new | (uintptr_t)d_o | (uintptr_t)d_cache_k |
                    (uintptr_t)d_cache_v | (uintptr_t)d_workspace) % 16 == 0, "pointers must be 16-byte aligned");
    NATS_CHECK_ARG(fill >= 0 && fill < C, "fill %d must lie in [0, chunk size %d)", fill, C);
    NATS_CHECK_ARG(max_len_bound >= SW && max_len_bound + fill < Lcap,
                   "length bound %d (+ fill %d) does not fit the cache capacity %d", max_len_bound, fill, Lcap);
    NATS_CHECK_ARG(B <= 65535 && Hkv <= 65535, "B and Hkv must not exceed 65535");
    const int nrep = Hq / Hkv;
    if (!(D == 64 || D == 128) || nrep > kMaxRep)
        return fail(NATS_ERR_UNSUPPORTED, "decode supports head_dim {64,128} and up to %d query heads per kv-head; got %d, %d",
                    kMaxRep, D, nrep);
    const int max_len = max_len_bound + C;
    const size_t need = nats_b200_decode_workspace_bytes(B, Hq, Hkv, D, max_len);
    if (workspace_bytes < need) return fail(NATS_ERR_WORKSPACE, "decode workspace: %zu bytes given, %zu needed", workspace_bytes, need);
    DecodeParams p;
    p.q = (const __nv_bfloat16*)d_q; p.k_new = (const __nv_bfloat16*)d_k_new; p.v_new = (const __nv_bfloat16*)d_v_new;
    p.o = (__nv_bfloat16*)d_o; p.ck = (__nv_bfloat16*)d_cache_k; p.cv = (__nv_bfloat16*)d_cache_v; p.valid = d_valid;
    p.size_global = (const long long*)d_size_global; p.size_local = (const long long*)d_size_local; p.state = d_state;
    p.counters = (int32_t*)d_workspace;
    p.partials = (float*)((uint8_t*)d_workspace + decode_counter_bytes(B, Hkv));
    p.Hq = Hq; p.Hkv = Hkv; p.nrep = nrep; p.Lcap = Lcap; p.SW = SW; p.fill = fill; p.fill_from_state = fill_from_state;
    p.max_splits = decode_max_splits(max_len);
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    dim3 grid(cdiv(max_len_bound + fill + 1, kSeg), Hkv, B);
    cudaError_t e = (D == 64) ? launch_decode<64>(p, grid, (cudaStream_t)stream) : launch_decode<128>(p, grid, (cudaStream_t)stream);
    NATS_CHECK_CUDA(e);
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_decode_fwd(const void* d_q, const void* d_k_new, const void* d_v_new, void* d_o,
                                    void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                                    const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                                    int fill, int max_len_bound,
                                    int B, int Hq, int Hkv, int D, int C, int SW, float sm_scale,
                                    void* d_workspace, size_t workspace_bytes, void* stream) {
    return decode_impl(d_q, d_k_new, d_v_new, d_o, d_cache_k, d_cache_v, d_valid, Lcap, d_size_global, d_size_local, d_state,
                       fill, max_len_bound, 0, B, Hq, Hkv, D, C, SW, sm_scale, d_workspace, workspace_bytes, stream);
}

extern "C" __attribute__((visibility("default"))) int nats_b200_decode_step_fwd(const void* d_q, const void* d_k_new, const void* d_v_new, void* d_o,
                                         void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                                         const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                                         int max_len_bound, int B, int Hq, int Hkv, int D, int C, int SW, float sm_scale,
                                         void* d_workspace, size_t workspace_bytes, void* stream) {
    // the fill is read on the device: size everything for the largest one
    return decode_impl(d_q, d_k_new, d_v_new, d_o, d_cache_k, d_cache_v, d_valid, Lcap, d_size_global, d_size_local, d_state,
                       C - 1, max_len_bound, 1, B, Hq, Hkv, D, C, SW, sm_scale, d_workspace, workspace_bytes, stream);
}
