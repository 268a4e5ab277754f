// Decode attention over the compacted ragged cache: split-KV, GQA-aware, HBM-bound.
//
// One block owns kSeg consecutive tokens of the *logical* sequence of one (batch, kv-head):
//     [ valid ring slots | kept tokens [SW,len) | tokens of the unfinished chunk [T0,T0+fill) | the new token ]
// A K or V row (D bf16) is read once, by D/8 lanes with one 16-byte load each, and serves all query heads of the
// group; dot products are reduced across those lanes with a reduce-scatter butterfly so that each lane finishes one
// (row, head) score, applies the online softmax to it and broadcasts the probability back for the P.V update.
// Blocks of a (batch, kv-head) leave partial (max, sum, acc) in the workspace; the block that arrives last combines
// them (an atomic ticket, nobody waits).  The block owning the last logical token also appends it to the cache.
#include "common.cuh"

namespace nats {

constexpr int kSeg = 512;          // logical tokens per block
constexpr int kDecThreads = 128;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kDecStages = 3;       // ring depth per warp: two iterations of loads in flight while one is consumed

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
    float* partials;               // [B*Hkv, max_splits, NREP, D+2]   (workspace)
    int Hq, Hkv, Lcap, SW, fill, max_splits;
    float scale_log2;              // sm_scale * log2(e)
};

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
    f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xffff0000u);
    f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xffff0000u);
    f[4] = __uint_as_float(w.z << 16); f[5] = __uint_as_float(w.z & 0xffff0000u);
    f[6] = __uint_as_float(w.w << 16); f[7] = __uint_as_float(w.w & 0xffff0000u);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16-byte asynchronous global -> shared copy that bypasses L1; with valid == false nothing is read and zeros are written
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D, int NREP, int U>
__global__ void __launch_bounds__(kDecThreads) decode_kernel(const DecodeParams p) {
    constexpr int TPR = D / 8;                       // lanes per row
    constexpr int RPW = 32 / TPR;                    // rows per warp per pass
    constexpr int V = U * NREP;                      // scores per lane group and iteration
    constexpr bool FAST = (V % TPR == 0) && (V / TPR <= NREP);
    constexpr int R = FAST ? V / TPR : V;            // scores finished by one lane
    constexpr int ROWS_IT = kDecWarps * RPW * U;
    constexpr int G = kDecWarps * RPW;               // lane groups per block
    constexpr unsigned FULL = 0xffffffffu;
    const float NEG_INF = -INFINITY;

    const int seg = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const int bh = b * p.Hkv + hkv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = lane % TPR, grp = lane / TPR;
    const int len = (int)(p.size_global[bh] + p.size_local[bh]);
    const int T0 = p.state[0];
    const int Ltot = len + p.fill + 1;
    const int nsplit = (Ltot + kSeg - 1) / kSeg;
    if (seg >= nsplit) return;
    const int r0 = seg * kSeg, r1 = min(Ltot, r0 + kSeg);

    // Dynamic shared memory: per warp a ring of kDecStages stages; a stage holds, for each of the U passes, the 16 bytes of
    // K and of V every lane has asked for (cp.async), so the bytes in flight do not occupy registers.  Each lane only ever
    // reads back what it copied itself, so cp.async.wait_group is the only synchronisation.  After the main loop the
    // same memory holds the per-lane-group partial results that are combined across the block.
    extern __shared__ __align__(16) uint8_t dsm[];
    constexpr int STAGE_BYTES = U * 2 * 32 * 16;
    constexpr int RING_BYTES = kDecWarps * kDecStages * STAGE_BYTES;
    constexpr int COMBINE_BYTES = G * NREP * (D + 2) * 4;
    static_assert(COMBINE_BYTES <= RING_BYTES, "combine scratch must fit into the ring");
    uint8_t* ring = dsm + warp * kDecStages * STAGE_BYTES + lane * 16;
    float (*s_acc)[NREP][D] = reinterpret_cast<float (*)[NREP][D]>(dsm);
    float (*s_m)[NREP] = reinterpret_cast<float (*)[NREP]>(dsm + G * NREP * D * 4);
    float (*s_l)[NREP] = reinterpret_cast<float (*)[NREP]>(dsm + G * NREP * (D + 1) * 4);
    __shared__ uint8_t s_ring_ok[kSeg];
    __shared__ int s_last;

    const size_t row_elems = (size_t)D;
    const __nv_bfloat16* ck = p.ck + (size_t)bh * p.Lcap * row_elems;
    const __nv_bfloat16* cv = p.cv + (size_t)bh * p.Lcap * row_elems;
    const uint8_t* valid = p.valid + (size_t)bh * p.Lcap;
    const __nv_bfloat16* kn = p.k_new + (size_t)bh * row_elems;
    const __nv_bfloat16* vn = p.v_new + (size_t)bh * row_elems;

    if (r0 < p.SW) {
        for (int i = tid; i < kSeg; i += kDecThreads) s_ring_ok[i] = (r0 + i < p.SW) ? valid[r0 + i] : 1;
    }
    // the block that owns the last logical token appends it (nobody reads that cache row in this launch)
    if (r1 == Ltot && warp == 0 && grp == 0) {
        const size_t dst = (size_t)(T0 + p.fill) * row_elems + j * 8;
        st16(p.ck + (size_t)bh * p.Lcap * row_elems + dst, ld16(kn + j * 8));
        st16(p.cv + (size_t)bh * p.Lcap * row_elems + dst, ld16(vn + j * 8));
        if (j == 0) p.valid[(size_t)bh * p.Lcap + T0 + p.fill] = 1;
    }
    // query fragments: this lane's 8 dims of every head of the group, pre-scaled
    float q[NREP][8];
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        const uint4 w = ld16(p.q + ((size_t)b * p.Hq + (size_t)hkv * NREP + h) * row_elems + j * 8);
        unpack8(w, q[h]);
#pragma unroll
        for (int d = 0; d < 8; ++d) q[h][d] *= p.scale_log2;
    }
    if (r0 < p.SW) __syncthreads();

    float acc[NREP][8];
#pragma unroll
    for (int h = 0; h < NREP; ++h)
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[h][d] = 0.f;
    float m_own[R], l_own[R];
#pragma unroll
    for (int r = 0; r < R; ++r) { m_own[r] = NEG_INF; l_own[r] = 0.f; }

    // issue the copies of iteration `it` into its ring stage (rows that do not exist or are invalid are zero-filled)
    auto issue = [&](int it) {
        const int base = r0 + it * ROWS_IT;
        uint8_t* dst = ring + (it % kDecStages) * STAGE_BYTES;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * (kDecWarps * RPW) + warp * RPW + grp;
            bool ok = i < r1;
            const __nv_bfloat16 *kp = ck, *vpp = cv;
            if (ok) {
                if (i < p.SW) { ok = s_ring_ok[i - r0] != 0; kp = ck + (size_t)i * row_elems; vpp = cv + (size_t)i * row_elems; }
                else if (i < len) { kp = ck + (size_t)i * row_elems; vpp = cv + (size_t)i * row_elems; }
                else if (i < len + p.fill) { const size_t ph = (size_t)(T0 + (i - len)); kp = ck + ph * row_elems; vpp = cv + ph * row_elems; }
                else { kp = kn; vpp = vn; }
            }
            cp_async16(dst + (u * 2 + 0) * 512, kp + j * 8, ok);
            cp_async16(dst + (u * 2 + 1) * 512, vpp + j * 8, ok);
        }
    };
    const int n_it = (r1 - r0 + ROWS_IT - 1) / ROWS_IT;
#pragma unroll
    for (int it = 0; it < kDecStages - 1; ++it) {
        if (it < n_it) issue(it);
        cp_async_commit();
    }
    for (int it = 0; it < n_it; ++it) {
        if (it + kDecStages - 1 < n_it) issue(it + kDecStages - 1);
        cp_async_commit();
        cp_async_wait<kDecStages - 1>();
        const int base = r0 + it * ROWS_IT;
        const uint8_t* src = ring + (it % kDecStages) * STAGE_BYTES;
        uint4 kq[U], vq[U];
        unsigned okmask = 0;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * (kDecWarps * RPW) + warp * RPW + grp;
            const bool ok = i < r1 && (i >= p.SW || s_ring_ok[i - r0] != 0);
            okmask |= (ok ? 1u : 0u) << u;
            kq[u] = *reinterpret_cast<const uint4*>(src + (u * 2 + 0) * 512);
            vq[u] = *reinterpret_cast<const uint4*>(src + (u * 2 + 1) * 512);
        }

        float part[V];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float kf[8];
            unpack8(kq[u], kf);
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                float s = 0.f;
#pragma unroll
                for (int d = 0; d < 8; ++d) s = fmaf(q[h][d], kf[d], s);
                part[u * NREP + h] = s;
            }
        }
        float p_all[V], alpha[NREP];
        if constexpr (FAST) {
            // reduce-scatter over the TPR lanes of the row: lane j ends with the totals of scores j*R .. j*R+R-1
            int cnt = V;
#pragma unroll
            for (int off = TPR / 2; off >= 1; off >>= 1) {
                cnt >>= 1;
                const bool upper = (j & off) != 0;
#pragma unroll
                for (int i = 0; i < V / 2; ++i) {
                    if (i < cnt) {
                        const float send = upper ? part[i] : part[i + cnt];
                        const float keep = upper ? part[i + cnt] : part[i];
                        part[i] = keep + __shfl_xor_sync(FULL, send, off);
                    }
                }
            }
            float pr[R], al[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int idx = j * R + r;
                const int u = idx / NREP;
                float s = ((okmask >> u) & 1u) ? part[r] : NEG_INF;
                float mt = s;                       // max over the U rows of this iteration, same head
#pragma unroll
                for (int off = NREP / R; off < TPR; off <<= 1) mt = fmaxf(mt, __shfl_xor_sync(FULL, mt, off));
                const float m_new = fmaxf(m_own[r], mt);
                const float m_use = (m_new == NEG_INF) ? 0.f : m_new;
                al[r] = fast_exp2(m_own[r] - m_use);
                pr[r] = fast_exp2(s - m_use);
                l_own[r] = l_own[r] * al[r] + pr[r];
                m_own[r] = m_new;
            }
            const int gbase = grp * TPR;
#pragma unroll
            for (int h = 0; h < NREP; ++h) alpha[h] = __shfl_sync(FULL, al[h % R], gbase + h / R);
#pragma unroll
            for (int i = 0; i < V; ++i) p_all[i] = __shfl_sync(FULL, pr[i % R], gbase + i / R);
        } else {
            // all-reduce every score; every lane then runs the same softmax update (R == V)
#pragma unroll
            for (int i = 0; i < V; ++i)
#pragma unroll
                for (int off = TPR / 2; off >= 1; off >>= 1) part[i] += __shfl_xor_sync(FULL, part[i], off);
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                float mt = NEG_INF;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (!((okmask >> u) & 1u)) part[u * NREP + h] = NEG_INF;
                    mt = fmaxf(mt, part[u * NREP + h]);
                }
                const float m_new = fmaxf(m_own[h], mt);        // slots 0..NREP-1 of m_own / l_own are per head here
                const float m_use = (m_new == NEG_INF) ? 0.f : m_new;
                alpha[h] = fast_exp2(m_own[h] - m_use);
                float ls = 0.f;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    p_all[u * NREP + h] = fast_exp2(part[u * NREP + h] - m_use);
                    ls += p_all[u * NREP + h];
                }
                l_own[h] = l_own[h] * alpha[h] + ls;
                m_own[h] = m_new;
            }
        }
#pragma unroll
        for (int h = 0; h < NREP; ++h)
#pragma unroll
            for (int d = 0; d < 8; ++d) acc[h][d] *= alpha[h];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float vf[8];
            unpack8(vq[u], vf);
#pragma unroll
            for (int h = 0; h < NREP; ++h)
#pragma unroll
                for (int d = 0; d < 8; ++d) acc[h][d] = fmaf(p_all[u * NREP + h], vf[d], acc[h][d]);
        }
    }

    // ---- combine the lane groups of this block (the ring is drained: every copy was waited for) ----
    cp_async_wait<0>();
    __syncthreads();
    const int g = warp * RPW + grp;
    if constexpr (FAST) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float l = l_own[r];
#pragma unroll
            for (int off = NREP / R; off < TPR; off <<= 1) l += __shfl_xor_sync(FULL, l, off);
            const int idx = j * R + r;
            if (idx < NREP) { s_m[g][idx] = m_own[r]; s_l[g][idx] = l; }
        }
    } else {
        if (j == 0) {
#pragma unroll
            for (int h = 0; h < NREP; ++h) { s_m[g][h] = m_own[h]; s_l[g][h] = l_own[h]; }
        }
    }
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        *reinterpret_cast<float4*>(&s_acc[g][h][j * 8]) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
        *reinterpret_cast<float4*>(&s_acc[g][h][j * 8 + 4]) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
    }
    __syncthreads();
    constexpr int PSTRIDE = D + 2;
    float* part_out = p.partials + ((size_t)bh * p.max_splits + seg) * NREP * PSTRIDE;
    for (int idx = tid; idx < NREP * D; idx += kDecThreads) {
        const int h = idx / D, d = idx % D;
        float mf = NEG_INF;
#pragma unroll
        for (int gg = 0; gg < G; ++gg) mf = fmaxf(mf, s_m[gg][h]);
        const float mu = (mf == NEG_INF) ? 0.f : mf;
        float a = 0.f, l = 0.f;
#pragma unroll
        for (int gg = 0; gg < G; ++gg) {
            const float w = fast_exp2(s_m[gg][h] - mu);
            a = fmaf(s_acc[gg][h][d], w, a);
            l = fmaf(s_l[gg][h], w, l);
        }
        if (nsplit == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            p.o[((size_t)b * p.Hq + (size_t)hkv * NREP + h) * D + d] = __float2bfloat16_rn(a * inv);
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
    const float* parts = p.partials + (size_t)bh * p.max_splits * NREP * PSTRIDE;
    for (int idx = tid; idx < NREP * D; idx += kDecThreads) {
        const int h = idx / D, d = idx % D;
        float mf = NEG_INF;
        for (int s = 0; s < nsplit; ++s) mf = fmaxf(mf, __ldcg(parts + ((size_t)s * NREP + h) * PSTRIDE + D));
        const float mu = (mf == NEG_INF) ? 0.f : mf;
        float a = 0.f, l = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float* ps = parts + ((size_t)s * NREP + h) * PSTRIDE;
            const float w = fast_exp2(__ldcg(ps + D) - mu);
            a = fmaf(__ldcg(ps + d), w, a);
            l = fmaf(__ldcg(ps + D + 1), w, l);
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        p.o[((size_t)b * p.Hq + (size_t)hkv * NREP + h) * D + d] = __float2bfloat16_rn(a * inv);
    }
    if (tid == 0) p.counters[bh] = 0;
}

template <int D, int NREP>
static cudaError_t launch_decode(const DecodeParams& p, dim3 grid, cudaStream_t st) {
    constexpr int TPR = D / 8;
    constexpr int U = (NREP * 4 >= TPR) ? 4 : ((NREP * 8 >= TPR) ? 8 : 4);
    constexpr int smem = kDecWarps * kDecStages * U * 2 * 32 * 16;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(decode_kernel<D, NREP, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    decode_kernel<D, NREP, U><<<grid, kDecThreads, smem, st>>>(p);
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

extern "C" __attribute__((visibility("default"))) int nats_b200_decode_fwd(const void* d_q, const void* d_k_new, const void* d_v_new, void* d_o,
                                    void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                                    const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                                    int fill, int max_len_bound,
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
    if (!(D == 64 || D == 128) || !(nrep == 1 || nrep == 2 || nrep == 4 || nrep == 8))
        return fail(NATS_ERR_UNSUPPORTED, "decode supports head_dim {64,128} and group size {1,2,4,8}; got %d, %d", D, nrep);
    const int max_len = max_len_bound + C;
    const size_t need = nats_b200_decode_workspace_bytes(B, Hq, Hkv, D, max_len);
    if (workspace_bytes < need) return fail(NATS_ERR_WORKSPACE, "decode workspace: %zu bytes given, %zu needed", workspace_bytes, need);
    DecodeParams p;
    p.q = (const __nv_bfloat16*)d_q; p.k_new = (const __nv_bfloat16*)d_k_new; p.v_new = (const __nv_bfloat16*)d_v_new;
    p.o = (__nv_bfloat16*)d_o; p.ck = (__nv_bfloat16*)d_cache_k; p.cv = (__nv_bfloat16*)d_cache_v; p.valid = d_valid;
    p.size_global = (const long long*)d_size_global; p.size_local = (const long long*)d_size_local; p.state = d_state;
    p.counters = (int32_t*)d_workspace;
    p.partials = (float*)((uint8_t*)d_workspace + decode_counter_bytes(B, Hkv));
    p.Hq = Hq; p.Hkv = Hkv; p.Lcap = Lcap; p.SW = SW; p.fill = fill;
    p.max_splits = decode_max_splits(max_len);
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    dim3 grid(cdiv(max_len_bound + fill + 1, kSeg), Hkv, B);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
#define NATS_DEC(DD, RR) if (D == DD && nrep == RR) e = launch_decode<DD, RR>(p, grid, st); else
    NATS_DEC(128, 1) NATS_DEC(128, 2) NATS_DEC(128, 4) NATS_DEC(128, 8)
    NATS_DEC(64, 1) NATS_DEC(64, 2) NATS_DEC(64, 4) NATS_DEC(64, 8)
    e = cudaErrorInvalidValue;
#undef NATS_DEC
    NATS_CHECK_CUDA(e);
    return NATS_OK;
}
