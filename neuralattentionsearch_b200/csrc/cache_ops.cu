// Role-mask metadata, eviction (keep-set ranks + stream compaction) and decode-step chunk placement.
// All of it is integer / byte work bounded by HBM traffic and launch latency: one block per (batch, kv-head)
// for the scans, 16-byte vectorised row copies for the data movement.
#include <stdarg.h>

#include "common.cuh"

namespace nats {

// ---- host-side error text ---------------------------------------------------------------------
static thread_local char g_err[512] = "";
char* last_error_buf() { return g_err; }
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

constexpr int kScanThreads = 256;

// =================================================================================================
// role_prep: per-chunk row limit, per-tile max/min limit, kept-tile count
// =================================================================================================
// Row limits of Nc chunks whose first token sits at position pos0: lim[c] = last query position that may see chunk c.
// Next-global index by a reversed inclusive min-scan, 256 chunks at a time from the end of the sequence; the last chunk
// counts as global.  *first_gf receives the index of the first global (or last) chunk.  All threads of the block call.
__device__ void scan_role_limits(const uint8_t* __restrict__ roles, int Nc, int C, int SW, int pos0,
                                 int32_t* __restrict__ lim, int* s, int* carry, int* first_gf) {
    const int tid = threadIdx.x;
    if (tid == 0) *carry = Nc - 1;
    __syncthreads();
    for (int hi = Nc; hi > 0; hi -= kScanThreads) {
        const int c = hi - 1 - tid;
        const int role = (c >= 0) ? roles[c] : NATS_ROLE_LOCAL;
        const bool gf = c >= 0 && (role == NATS_ROLE_GLOBAL || c == Nc - 1);
        s[tid] = gf ? c : kNoLimit;
        __syncthreads();
        for (int o = 1; o < kScanThreads; o <<= 1) {
            const int v = (tid >= o) ? s[tid - o] : kNoLimit;
            __syncthreads();
            s[tid] = min(s[tid], v);
            __syncthreads();
        }
        const int fill = min(s[tid], *carry);
        if (c >= 0) {
            long long l;
            if (role == NATS_ROLE_SLIDING) l = (long long)pos0 + (long long)c * C + SW + C - 1;
            else if (gf) l = kNoLimit;
            else l = (long long)pos0 + ((long long)fill + 1) * C - 1;
            lim[c] = (int)min(l, (long long)kNoLimit);
            if (c == 0) *first_gf = fill;
        }
        __syncthreads();
        if (tid == kScanThreads - 1) *carry = fill;
        __syncthreads();
    }
}

// Per 128-row KV tile: max / min of the limits of the chunks it overlaps, and how many query tiles keep it.  Query row i
// sits at position q_off + i; there are Nt query tiles of 128 rows.  Returns this thread's share of the kept count.
__device__ unsigned long long tile_limits(const int32_t* __restrict__ lim, int Nkv, int C, int Ntk, int q_off, int Nt,
                                          int32_t* __restrict__ tmax, int32_t* __restrict__ tmin) {
    unsigned long long mine = 0;
    for (int kt = threadIdx.x; kt < Ntk; kt += kScanThreads) {
        const int c0 = (int)(((long long)kt * kTile) / C);
        const int c1 = (int)(min((long long)kt * kTile + kTile - 1, (long long)Nkv - 1) / C);
        int mx = -1, mn = kNoLimit;
        for (int c = c0; c <= c1; ++c) {
            const int l = lim[c];
            mx = max(mx, l);
            mn = min(mn, l);
        }
        tmax[kt] = mx;
        tmin[kt] = mn;
        // query tiles t that keep the tile: last row position >= first tile row, first row position <= mx
        const long long first = (long long)kt * kTile - q_off - (kTile - 1);
        const int t_min = first <= 0 ? 0 : (int)((first + kTile - 1) / kTile);
        if (mx >= q_off) {
            const int t_max = min(Nt - 1, (mx - q_off) / kTile);
            if (t_max >= t_min) mine += (unsigned long long)(t_max - t_min + 1);
        }
    }
    return mine;
}

__global__ void __launch_bounds__(kScanThreads)
role_prep_kernel(const uint8_t* __restrict__ roles, int Nc, int N, int C, int SW, int Nt,
                 int32_t* __restrict__ lim, int32_t* __restrict__ tmax, int32_t* __restrict__ tmin,
                 long long* __restrict__ kept) {
    const int bh = blockIdx.x, tid = threadIdx.x;
    roles += (size_t)bh * Nc;
    lim += (size_t)bh * Nc;
    tmax += (size_t)bh * Nt;
    tmin += (size_t)bh * Nt;
    __shared__ int s[kScanThreads];
    __shared__ int carry, first_gf;
    __shared__ unsigned long long kept_sm;
    if (tid == 0) kept_sm = 0;
    scan_role_limits(roles, Nc, C, SW, 0, lim, s, &carry, &first_gf);
    const unsigned long long mine = tile_limits(lim, N, C, Nt, 0, Nt, tmax, tmin);
    if (kept != nullptr) {
        atomicAdd(&kept_sm, mine);
        __syncthreads();
        if (tid == 0) kept[bh] = (long long)kept_sm;
    }
}

// The same metadata for a multi-token call over an existing cache.  The KV sequence is the physical cache layout
// [ring | kept global | kept local | gap | unfinished chunk + new tokens]; T0 = first position of the unfinished chunk.
struct PastPrepParams {
    const uint8_t* roles;                       // [BH, Ncn] roles of the chunks from the unfinished one on
    const uint8_t* valid;                       // [BH, Lcap]; only the ring flags [0, SW) of a head are read
    const long long* size_global; const long long* size_local;
    int32_t* lim; int32_t* tmax; int32_t* tmin; long long* kept;
    int Ncn, Lcap, T0, C, SW, tail, Nq, q_off, Nkv, Nc, Ntk, Nt;
};

__global__ void __launch_bounds__(kScanThreads) role_prep_past_kernel(const PastPrepParams p) {
    const int bh = blockIdx.x, tid = threadIdx.x;
    const uint8_t* roles = p.roles + (size_t)bh * p.Ncn;
    const uint8_t* valid = p.valid + (size_t)bh * p.Lcap;
    int32_t* lim = p.lim + (size_t)bh * p.Nc;
    __shared__ int s[kScanThreads];
    __shared__ int carry, first_gf;
    __shared__ unsigned long long kept_sm;
    if (tid == 0) kept_sm = 0;
    const int n_old = p.T0 / p.C, W = p.SW / p.C;
    // new chunks: the rule of a first call, positions counted from T0
    scan_role_limits(roles, p.Ncn, p.C, p.SW, p.T0, lim + n_old, s, &carry, &first_gf);
    // cached chunks
    const int sg = (int)(p.size_global[bh] / p.C), sl = (int)(p.size_local[bh] / p.C);
    const long long lim_local = (long long)p.T0 + ((long long)first_gf + 1) * p.C - 1;   // until the first new global chunk ends
    for (int j = tid; j < n_old; j += kScanThreads) {
        int l;
        if (j < W) {
            // ring slot j was written `age` chunks before the newest one; a sliding chunk is seen by the SW/C chunks after it
            const int age = ((p.tail / p.C - 1 - j) % W + W) % W;
            l = valid[(size_t)j * p.C] ? p.T0 + (W - age) * p.C - 1 : -1;
        } else if (j < sg) {
            l = kNoLimit;
        } else if (j < sg + sl) {
            l = (int)min(lim_local, (long long)kNoLimit);
        } else {
            l = -1;                                   // between this head's length and the longest head's
        }
        lim[j] = l;
    }
    __syncthreads();
    const unsigned long long mine = tile_limits(lim, p.Nkv, p.C, p.Ntk, p.q_off, p.Nt,
                                                p.tmax + (size_t)bh * p.Ntk, p.tmin + (size_t)bh * p.Ntk);
    if (p.kept != nullptr) {
        atomicAdd(&kept_sm, mine);
        __syncthreads();
        if (tid == 0) p.kept[bh] = (long long)kept_sm;
    }
}

// Number of keys every query row may see (first call): sum over the chunks in front of the row.  One thread per row of a
// kv-head; the count is written for each query head of the group.
__global__ void __launch_bounds__(kScanThreads)
visible_count_kernel(const int32_t* __restrict__ lim, int Hq, int Hkv, int N, int C, int Nc, int32_t* __restrict__ out) {
    const int bh = blockIdx.y;
    const int q = blockIdx.x * kScanThreads + threadIdx.x;
    if (q >= N) return;
    lim += (size_t)bh * Nc;
    const int c_last = q / C;
    int n = 0;
    for (int c = 0; c <= c_last; ++c)
        if (q <= lim[c]) n += min(q - c * C + 1, C);
    const int nrep = Hq / Hkv, b = bh / Hkv, hkv = bh % Hkv;
    for (int r = 0; r < nrep; ++r) out[((size_t)b * Hq + hkv * nrep + r) * N + q] = n;
}

// =================================================================================================
// evict_plan: keep flags -> destination ranks (ballot + prefix sum), sizes, max length
// =================================================================================================
__device__ __forceinline__ void publish_max_len(int32_t* state, int len, int nblocks) {
    // state[1] accumulates the maximum over blocks; the last block to arrive publishes it in state[0]
    // and leaves the scratch words zero for the next call.  No block ever waits for another.
    __shared__ int last;
    if (threadIdx.x == 0) {
        atomicMax(&state[1], len);
        __threadfence();
        const int ticket = atomicAdd(&state[2], 1);
        last = (ticket == nblocks - 1);
        if (last) {
            __threadfence();
            const int m = atomicExch(&state[1], 0);
            state[0] = m;
            state[2] = 0;
        }
    }
}

// base == nullptr: first call (the cache is empty: sizes are outputs).  Otherwise the sizes are read and updated, and
// base[bh] receives the chunk slot (counted from position 0) the first kept chunk of this call goes to: behind the
// kept locals if the call brings no global chunk, else behind the kept globals (the locals in front of it are dropped).
__global__ void __launch_bounds__(kScanThreads)
evict_plan_kernel(const uint8_t* __restrict__ roles, int Nc, int n_full, int C, int SW,
                  int32_t* __restrict__ rank, long long* __restrict__ size_global,
                  long long* __restrict__ size_local, int32_t* __restrict__ state, int32_t* __restrict__ base) {
    const int bh = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    roles += (size_t)bh * Nc;
    rank += (size_t)bh * Nc;
    __shared__ int s_last_g;
    __shared__ int s_warp[kScanThreads / 32];
    __shared__ int s_base, s_ng;
    if (tid == 0) { s_last_g = -1; s_base = 0; s_ng = 0; }
    __syncthreads();
    // pass 1: last global chunk among the complete chunks
    int lg = -1;
    for (int c = tid; c < n_full; c += kScanThreads)
        if (roles[c] == NATS_ROLE_GLOBAL) lg = c;
    for (int o = 16; o > 0; o >>= 1) lg = max(lg, __shfl_xor_sync(0xffffffffu, lg, o));
    if (lane == 0 && lg >= 0) atomicMax(&s_last_g, lg);
    __syncthreads();
    const int last_g = s_last_g;
    // pass 2: ordered ranks of the kept chunks
    for (int c0 = 0; c0 < Nc; c0 += kScanThreads) {
        const int c = c0 + tid;
        const int role = (c < n_full) ? roles[c] : -1;
        const bool is_g = role == NATS_ROLE_GLOBAL;
        const bool keep = is_g || (role == NATS_ROLE_LOCAL && c > last_g);
        const unsigned m = __ballot_sync(0xffffffffu, keep);
        const unsigned mg = __ballot_sync(0xffffffffu, is_g);
        if (lane == 0) s_warp[warp] = __popc(m);
        if (lane == 0 && mg) atomicAdd(&s_ng, __popc(mg));
        __syncthreads();
        int before = s_base;
        for (int w = 0; w < warp; ++w) before += s_warp[w];
        // kept chunk: its rank; other chunks: -1 - (kept chunks in front of it), so that the number of kept chunks up to any
        // index can be read off without a scan (the compaction finds the chunk of a given rank by bisection)
        const int kept_before = before + __popc(m & ((1u << lane) - 1u));
        if (c < Nc) rank[c] = keep ? kept_before : -1 - kept_before;
        __syncthreads();
        if (tid == 0) {
            int tot = 0;
            for (int w = 0; w < kScanThreads / 32; ++w) tot += s_warp[w];
            s_base += tot;
        }
        __syncthreads();
    }
    const int n_kept = s_base, n_g = s_ng;
    long long sg0 = SW, sl0 = 0;
    if (base != nullptr) { sg0 = size_global[bh]; sl0 = size_local[bh]; }
    const long long sg = sg0 + (long long)C * n_g;
    const long long sl = (last_g >= 0 ? 0 : sl0) + (long long)C * (n_kept - n_g);
    if (tid == 0) {
        size_global[bh] = sg;
        size_local[bh] = sl;
        if (base != nullptr) base[bh] = (int)((last_g >= 0 ? sg0 : sg0 + sl0) / C);
    }
    publish_max_len(state, (int)(sg + sl), gridDim.x);
}

// =================================================================================================
// evict_compact: ring fill + kept-chunk copies + pending tail + zero / valid bookkeeping
// =================================================================================================
constexpr int kCopyThreads = 256;
constexpr int kTokPerBlock = 64;

struct CompactParams {
    // source of the tokens of this call: [BH, src_stride, rowB] bytes; token t of the call sits at row src_off + t.
    // First call: the caller's K/V (src_off 0).  Call over an existing cache: the old cache buffer, to which the new
    // tokens were appended behind the unfinished chunk (src_off = old T0); it also holds the old ring and kept region.
    const uint8_t* k; const uint8_t* v; const uint8_t* old_valid;
    const uint8_t* roles; const int32_t* rank;   // [BH, Nc]
    const int32_t* base;                         // [BH] or nullptr (first call: SW / C)
    const long long* size_global; const long long* size_local; const int32_t* state;
    uint8_t* ck; uint8_t* cv; uint8_t* valid;    // [BH, Lcap, rowB], [BH, Lcap]
    long long src_stride;                        // rows per head of the source
    int src_off, tail, N, Nc, n_full, C, SW, Lcap, rowB;        // rowB = D * 2 bytes; N = tokens of the call
    int nB;                                      // blocks of the ring section
};

__global__ void __launch_bounds__(kCopyThreads) evict_compact_kernel(const CompactParams p) {
    const int bh = blockIdx.y, tid = threadIdx.x;
    const int vpt = p.rowB >> 4;                          // 16-byte vectors per token row
    const int tpp = kCopyThreads / vpt;                   // tokens per pass
    const int trow = tid / vpt, tvec = (tid % vpt) << 4;
    const uint8_t* k = p.k + (size_t)bh * p.src_stride * p.rowB;
    const uint8_t* v = p.v + (size_t)bh * p.src_stride * p.rowB;
    uint8_t* ck = p.ck + (size_t)bh * p.Lcap * p.rowB;
    uint8_t* cv = p.cv + (size_t)bh * p.Lcap * p.rowB;
    uint8_t* valid = p.valid + (size_t)bh * p.Lcap;
    const uint8_t* roles = p.roles + (size_t)bh * p.Nc;
    const int32_t* rank = p.rank + (size_t)bh * p.Nc;
    const bool past = p.base != nullptr;
    const int base = past ? p.base[bh] : p.SW / p.C;      // chunk slot of the first kept chunk of this call
    const uint4 zero = make_uint4(0, 0, 0, 0);
    int blk = blockIdx.x;
    if (blk < p.nB) {
        if (trow >= tpp) return;                          // head dims whose vector count does not divide 256
        // section B: the last min(n_full, SW/C) complete chunks of the call go to the ring slots behind the tail (data if
        // the chunk is a sliding one, else zeros + invalid); slots the call does not reach keep what they held
        const int n_upd = min(p.n_full, p.SW / p.C);
        const int n_fills = n_upd * p.C;
        const int src0 = (p.n_full - n_upd) * p.C;
        const int s0 = blk * kTokPerBlock;
        for (int i = trow; i < kTokPerBlock; i += tpp) {
            const int slot = s0 + i;
            if (slot >= p.SW) break;
            const int j = (slot - p.tail + p.SW) % p.SW;          // position in the write order of this call
            const size_t dst = (size_t)slot * p.rowB + tvec;
            if (j < n_fills) {
                const bool sw = roles[(src0 + j) / p.C] == NATS_ROLE_SLIDING;
                const size_t src = (size_t)(p.src_off + src0 + j) * p.rowB + tvec;
                st16(ck + dst, sw ? ld16_stream(k + src) : zero);
                st16(cv + dst, sw ? ld16_stream(v + src) : zero);
                if (tvec == 0) valid[slot] = sw ? 1 : 0;
            } else if (past) {
                st16(ck + dst, ld16_stream(k + dst));
                st16(cv + dst, ld16_stream(v + dst));
                if (tvec == 0) valid[slot] = p.old_valid[(size_t)bh * p.src_stride + slot];
            } else {
                st16(ck + dst, zero);
                st16(cv + dst, zero);
                if (tvec == 0) valid[slot] = 0;
            }
        }
        return;
    }
    blk -= p.nB;
    // main region, destination-driven.  [SW, base*C) = what the cache kept from before this call; [base*C, len) = the kept
    // chunks of this call (slot r holds the chunk whose rank is r: ranks grow with the chunk index, so the chunk is found
    // by bisection); [len, Lcap) is zero except the tokens of the unfinished chunk at [T0, T0+rem).  Launching blocks per
    // destination instead of per source token matters: most source chunks are not kept.
    // Step 1: one thread per destination token of the block works out where its row comes from (source row in k / v,
    // -1: zeros, -2: leave alone), so that the bisection's chain of dependent loads is paid once per block and not in front
    // of every copy.  Step 2: every thread loads all of its 16-byte vectors, then stores them.
    __shared__ int s_src[kTokPerBlock];
    const int len = (int)(p.size_global[bh] + p.size_local[bh]);
    const int T0 = p.state[0];
    const int rem = p.N - p.n_full * p.C;
    const int d0 = p.SW + blk * kTokPerBlock;
    if (tid < kTokPerBlock) {
        const int d = d0 + tid;
        int src = -2;
        if (d < p.Lcap) {
            const bool in_tail = d >= T0 && d < T0 + rem;
            valid[d] = (d < len || in_tail) ? 1 : 0;
            if (d < len) {
                if (d < base * p.C) {
                    if (past) src = d;
                } else {
                    // the chunk of rank r: the smallest index up to which r + 1 chunks are kept
                    const int r = d / p.C - base;
                    int lo = r, hi = p.n_full - 1;                 // it cannot sit in front of index r
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        const int v = rank[mid];
                        const int kept_upto = v >= 0 ? v + 1 : -1 - v;         // kept chunks in [0, mid]
                        if (kept_upto >= r + 1) hi = mid; else lo = mid + 1;
                    }
                    src = p.src_off + lo * p.C + d % p.C;
                }
            } else if (in_tail) {
                src = p.src_off + p.n_full * p.C + (d - T0);
            } else {
                src = -1;
            }
        }
        s_src[tid] = src;
    }
    __syncthreads();
    if (trow >= tpp) return;                              // head dims whose vector count does not divide 256
    constexpr int kBatch = 4;
    for (int i0 = trow; i0 < kTokPerBlock; i0 += kBatch * tpp) {
        uint4 a[kBatch], b[kBatch];
        int sr[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int i = i0 + u * tpp;
            sr[u] = i < kTokPerBlock ? s_src[i] : -2;
            a[u] = b[u] = zero;
            if (sr[u] >= 0) {
                const size_t src = (size_t)sr[u] * p.rowB + tvec;
                a[u] = ld16_stream(k + src);
                b[u] = ld16_stream(v + src);
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            if (sr[u] == -2) continue;
            const size_t dst = (size_t)(d0 + i0 + u * tpp) * p.rowB + tvec;
            st16(ck + dst, a[u]);
            st16(cv + dst, b[u]);
        }
    }
}

// Appends the K/V of new tokens to a cache buffer at row `pos` of every (b,h) and marks them valid.
struct AppendParams {
    const uint8_t* k; const uint8_t* v;          // [BH, x_len, rowB]
    uint8_t* ck; uint8_t* cv; uint8_t* valid;    // [BH, Lcap, rowB], [BH, Lcap]
    int x_len, pos, Lcap, rowB;
};

__global__ void __launch_bounds__(kCopyThreads) cache_append_kernel(const AppendParams p) {
    const int bh = blockIdx.y, tid = threadIdx.x;
    const int vpt = p.rowB >> 4, tpp = kCopyThreads / vpt;
    const int trow = tid / vpt, tvec = (tid % vpt) << 4;
    if (trow >= tpp) return;
    const uint8_t* k = p.k + (size_t)bh * p.x_len * p.rowB;
    const uint8_t* v = p.v + (size_t)bh * p.x_len * p.rowB;
    uint8_t* ck = p.ck + ((size_t)bh * p.Lcap + p.pos) * p.rowB;
    uint8_t* cv = p.cv + ((size_t)bh * p.Lcap + p.pos) * p.rowB;
    uint8_t* valid = p.valid + (size_t)bh * p.Lcap + p.pos;
    const int t0 = blockIdx.x * kTokPerBlock;
    for (int i = trow; i < kTokPerBlock; i += tpp) {
        const int t = t0 + i;
        if (t >= p.x_len) break;
        const size_t o = (size_t)t * p.rowB + tvec;
        st16(ck + o, ld16_stream(k + o));
        st16(cv + o, ld16_stream(v + o));
        if (tvec == 0) valid[t] = 1;
    }
}

// =================================================================================================
// decode_place: a chunk completed by decode steps goes to the ring and, unless sliding, behind the kept chunks
// =================================================================================================
struct PlaceParams {
    const uint8_t* roles;                         // [BH]
    uint8_t* ck; uint8_t* cv; uint8_t* valid;
    long long* size_global; long long* size_local; int32_t* state;
    int C, SW, Lcap, rowB, tail;
    int from_state;                               // 1: static launch -- act only if state[4] + 1 == C, ring position = state[5]
};

__global__ void __launch_bounds__(kCopyThreads) decode_place_kernel(const PlaceParams p) {
    const int bh = blockIdx.x, tid = threadIdx.x;
    const int vpt = p.rowB >> 4, tpp = kCopyThreads / vpt;
    const int trow = tid / vpt, tvec = (tid % vpt) << 4;
    uint8_t* ck = p.ck + (size_t)bh * p.Lcap * p.rowB;
    uint8_t* cv = p.cv + (size_t)bh * p.Lcap * p.rowB;
    uint8_t* valid = p.valid + (size_t)bh * p.Lcap;
    int tail = p.tail;
    if (p.from_state) {
        if (p.state[4] + 1 != p.C) return;        // the step did not complete a chunk (uniform for the grid)
        tail = p.state[5];
    }
    const int role = p.roles[bh];
    const int T0 = p.state[0];
    const long long sg = p.size_global[bh], sl = p.size_local[bh];
    const int len = (int)(sg + sl);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    int dst, new_len;
    long long nsg = sg, nsl = sl;
    if (role == NATS_ROLE_GLOBAL) { dst = (int)sg; nsg = sg + p.C; nsl = 0; }
    else if (role == NATS_ROLE_LOCAL) { dst = len; nsl = sl + p.C; }
    else { dst = -1; }
    new_len = (int)(nsg + nsl);
    if (trow < tpp) {
        for (int i = trow; i < p.C; i += tpp) {
            const size_t src = (size_t)(T0 + i) * p.rowB + tvec;
            const uint4 kk = ld16(ck + src), vv = ld16(cv + src);
            const int slot = (tail + i) % p.SW;
            const size_t rdst = (size_t)slot * p.rowB + tvec;
            const bool sw = role == NATS_ROLE_SLIDING;
            st16(ck + rdst, sw ? kk : zero);
            st16(cv + rdst, sw ? vv : zero);
            if (tvec == 0) valid[slot] = sw ? 1 : 0;
            if (dst >= 0 && dst != T0) {
                const size_t mdst = (size_t)(dst + i) * p.rowB + tvec;
                st16(ck + mdst, kk);
                st16(cv + mdst, vv);
            }
        }
    }
    __syncthreads();   // every read of the pending chunk is done before the region behind the new length is cleared
    if (trow < tpp) {
        // cleared: the locals a global chunk has just dropped, [new_len, len), and the slot of the pending chunk unless the
        // chunk stayed there; everything else behind a head's length is zero already
        for (int d = new_len + trow; d < len; d += tpp) {
            const size_t o = (size_t)d * p.rowB + tvec;
            st16(ck + o, zero);
            st16(cv + o, zero);
            if (tvec == 0) valid[d] = 0;
        }
        const int end = min(T0 + p.C, p.Lcap);
        for (int d = max(T0, new_len) + trow; d < end; d += tpp) {
            const size_t o = (size_t)d * p.rowB + tvec;
            st16(ck + o, zero);
            st16(cv + o, zero);
            if (tvec == 0) valid[d] = 0;
        }
        if (dst >= 0)
            for (int i = trow; i < p.C; i += tpp)
                if (tvec == 0) valid[dst + i] = 1;
    }
    if (tid == 0) {
        p.size_global[bh] = nsg;
        p.size_local[bh] = nsl;
    }
    publish_max_len(p.state, new_len, gridDim.x);
}

}  // namespace nats

// =================================================================================================
// C ABI
// =================================================================================================
using namespace nats;

extern "C" __attribute__((visibility("default"))) const char* nats_b200_last_error(void) { return last_error_buf(); }

extern "C" __attribute__((visibility("default"))) const char* nats_b200_build_info(void) {
    return "libnats_b200 sm_100a; prefill tile 128x128 (tcgen05/TMEM/TMA), head_dim {64,128}, N <= 524288; "
           "decode head_dim {64,128}, group size 1..8";
}

static int check_common(int B, int Hkv, int N, int C, int SW) {
    NATS_CHECK_ARG(B > 0 && Hkv > 0 && N > 0, "B, Hkv and N must be positive (got %d, %d, %d)", B, Hkv, N);
    NATS_CHECK_ARG(C > 0 && SW > 0 && SW % C == 0, "sliding window %d must be a positive multiple of the chunk size %d", SW, C);
    NATS_CHECK_ARG((long long)B * Hkv <= 65535, "B * Hkv = %lld exceeds the grid limit 65535", (long long)B * Hkv);
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_role_prep(const uint8_t* d_roles, int B, int Hkv, int N, int C, int SW,
                                   int32_t* d_lim, int32_t* d_tile_max, int32_t* d_tile_min, int64_t* d_kept_tiles,
                                   void* stream) {
    if (int rc = check_common(B, Hkv, N, C, SW)) return rc;
    NATS_CHECK_ARG(d_roles && d_lim && d_tile_max && d_tile_min, "null pointer");
    const int Nc = cdiv(N, C), Nt = cdiv(N, kTile);
    role_prep_kernel<<<B * Hkv, kScanThreads, 0, (cudaStream_t)stream>>>(
        d_roles, Nc, N, C, SW, Nt, d_lim, d_tile_max, d_tile_min, (long long*)d_kept_tiles);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_visible_counts(const int32_t* d_lim, int B, int Hq, int Hkv, int N, int C,
                                                                    int32_t* d_n_visible, void* stream) {
    NATS_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && N > 0 && C > 0 && Hq % Hkv == 0 && (long long)B * Hkv <= 65535,
                   "bad shape B=%d Hq=%d Hkv=%d N=%d C=%d", B, Hq, Hkv, N, C);
    NATS_CHECK_ARG(d_lim && d_n_visible, "null pointer");
    dim3 grid(cdiv(N, kScanThreads), B * Hkv);
    visible_count_kernel<<<grid, kScanThreads, 0, (cudaStream_t)stream>>>(d_lim, Hq, Hkv, N, C, cdiv(N, C), d_n_visible);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_evict_plan(const uint8_t* d_roles, int B, int Hkv, int N, int C, int SW,
                                    int32_t* d_rank, int64_t* d_size_global, int64_t* d_size_local, int32_t* d_state,
                                    void* stream) {
    if (int rc = check_common(B, Hkv, N, C, SW)) return rc;
    NATS_CHECK_ARG(d_roles && d_rank && d_size_global && d_size_local && d_state, "null pointer");
    const int Nc = cdiv(N, C);
    evict_plan_kernel<<<B * Hkv, kScanThreads, 0, (cudaStream_t)stream>>>(
        d_roles, Nc, N / C, C, SW, d_rank, (long long*)d_size_global, (long long*)d_size_local, d_state, nullptr);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_role_prep_past(
    const uint8_t* d_roles_new, const uint8_t* d_valid, const int64_t* d_size_global, const int64_t* d_size_local,
    int B, int Hkv, int x_len, int C, int SW, int valid_stride, int t0, int fill, int tail,
    int32_t* d_lim, int32_t* d_tile_max, int32_t* d_tile_min, int64_t* d_kept_tiles, void* stream) {
    if (int rc = check_common(B, Hkv, x_len, C, SW)) return rc;
    NATS_CHECK_ARG(d_roles_new && d_valid && d_size_global && d_size_local && d_lim && d_tile_max && d_tile_min, "null pointer");
    NATS_CHECK_ARG(t0 >= SW && t0 % C == 0 && fill >= 0 && fill < C, "tail offset %d must be a chunk multiple >= the window, fill %d in [0, chunk)", t0, fill);
    NATS_CHECK_ARG(tail >= 0 && tail < SW && tail % C == 0, "ring tail %d must be a chunk multiple inside the window %d", tail, SW);
    NATS_CHECK_ARG(valid_stride >= SW, "the flags of a head (%d) must cover the ring (%d)", valid_stride, SW);
    NATS_CHECK_ARG((long long)t0 + fill + x_len <= 0x7fffffffLL - 2 * (long long)(SW + C), "sequence too long");
    PastPrepParams p;
    p.roles = d_roles_new; p.valid = d_valid;
    p.size_global = (const long long*)d_size_global; p.size_local = (const long long*)d_size_local;
    p.lim = d_lim; p.tmax = d_tile_max; p.tmin = d_tile_min; p.kept = (long long*)d_kept_tiles;
    p.Ncn = cdiv(fill + x_len, C); p.Lcap = valid_stride; p.T0 = t0; p.C = C; p.SW = SW; p.tail = tail;
    p.Nq = x_len; p.q_off = t0 + fill; p.Nkv = t0 + fill + x_len;
    p.Nc = cdiv(p.Nkv, C); p.Ntk = cdiv(p.Nkv, kTile); p.Nt = cdiv(x_len, kTile);
    role_prep_past_kernel<<<B * Hkv, kScanThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_evict_plan_past(
    const uint8_t* d_roles_new, int B, int Hkv, int n_tokens, int C, int SW, int32_t* d_rank, int32_t* d_base,
    int64_t* d_size_global, int64_t* d_size_local, int32_t* d_state, void* stream) {
    if (int rc = check_common(B, Hkv, n_tokens, C, SW)) return rc;
    NATS_CHECK_ARG(d_roles_new && d_rank && d_base && d_size_global && d_size_local && d_state, "null pointer");
    evict_plan_kernel<<<B * Hkv, kScanThreads, 0, (cudaStream_t)stream>>>(
        d_roles_new, cdiv(n_tokens, C), n_tokens / C, C, SW, d_rank, (long long*)d_size_global, (long long*)d_size_local,
        d_state, d_base);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

static int check_row(int D) {
    NATS_CHECK_ARG(D > 0 && (D * 2) % 16 == 0 && D <= 2048 && 256 % ((D * 2) / 16) == 0,
                   "head_dim %d: a bf16 row must be a whole number of 16-byte vectors that divides 256", D);
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_evict_compact(const void* d_k, const void* d_v, const uint8_t* d_roles, const int32_t* d_rank,
                                       const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
                                       int B, int Hkv, int N, int D, int C, int SW,
                                       void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap, void* stream) {
    if (int rc = check_common(B, Hkv, N, C, SW)) return rc;
    if (int rc = check_row(D)) return rc;
    NATS_CHECK_ARG(d_k && d_v && d_roles && d_rank && d_size_global && d_size_local && d_state && d_cache_k && d_cache_v && d_valid,
                   "null pointer");
    NATS_CHECK_ARG(((uintptr_t)d_k | (uintptr_t)d_v | (uintptr_t)d_cache_k | (uintptr_t)d_cache_v) % 16 == 0,
                   "K/V and cache pointers must be 16-byte aligned");
    NATS_CHECK_ARG(Lcap >= SW + C, "cache capacity %d is smaller than ring + one chunk (%d)", Lcap, SW + C);
    CompactParams p;
    p.k = (const uint8_t*)d_k; p.v = (const uint8_t*)d_v; p.roles = d_roles; p.rank = d_rank;
    p.old_valid = nullptr; p.base = nullptr; p.src_stride = N; p.src_off = 0; p.tail = 0;
    p.size_global = (const long long*)d_size_global; p.size_local = (const long long*)d_size_local; p.state = d_state;
    p.ck = (uint8_t*)d_cache_k; p.cv = (uint8_t*)d_cache_v; p.valid = d_valid;
    p.N = N; p.Nc = cdiv(N, C); p.n_full = N / C; p.C = C; p.SW = SW; p.Lcap = Lcap; p.rowB = D * 2;
    p.nB = cdiv(SW, kTokPerBlock);
    const int nC = cdiv(Lcap - SW, kTokPerBlock);
    dim3 grid(p.nB + nC, B * Hkv);
    evict_compact_kernel<<<grid, kCopyThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_evict_compact_past(
    const void* d_old_k, const void* d_old_v, const uint8_t* d_old_valid, int old_capacity,
    const uint8_t* d_roles_new, const int32_t* d_rank, const int32_t* d_base,
    const int64_t* d_size_global, const int64_t* d_size_local, const int32_t* d_state,
    int B, int Hkv, int n_tokens, int D, int C, int SW, int t0_old, int tail_old,
    void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap, void* stream) {
    if (int rc = check_common(B, Hkv, n_tokens, C, SW)) return rc;
    if (int rc = check_row(D)) return rc;
    NATS_CHECK_ARG(d_old_k && d_old_v && d_old_valid && d_roles_new && d_rank && d_base && d_size_global && d_size_local &&
                   d_state && d_cache_k && d_cache_v && d_valid, "null pointer");
    NATS_CHECK_ARG(((uintptr_t)d_old_k | (uintptr_t)d_old_v | (uintptr_t)d_cache_k | (uintptr_t)d_cache_v) % 16 == 0,
                   "cache pointers must be 16-byte aligned");
    NATS_CHECK_ARG(d_old_k != d_cache_k && d_old_v != d_cache_v && d_old_valid != d_valid, "the compaction is out of place: old and new cache must differ");
    NATS_CHECK_ARG(t0_old >= SW && t0_old % C == 0 && (long long)t0_old + n_tokens <= old_capacity,
                   "old cache: tail offset %d (+ %d tokens) does not fit its capacity %d", t0_old, n_tokens, old_capacity);
    NATS_CHECK_ARG(tail_old >= 0 && tail_old < SW && tail_old % C == 0, "ring tail %d must be a chunk multiple inside the window %d", tail_old, SW);
    NATS_CHECK_ARG(Lcap >= SW + C, "cache capacity %d is smaller than ring + one chunk (%d)", Lcap, SW + C);
    CompactParams p;
    p.k = (const uint8_t*)d_old_k; p.v = (const uint8_t*)d_old_v; p.old_valid = d_old_valid; p.roles = d_roles_new; p.rank = d_rank;
    p.base = d_base; p.src_stride = old_capacity; p.src_off = t0_old; p.tail = tail_old;
    p.size_global = (const long long*)d_size_global; p.size_local = (const long long*)d_size_local; p.state = d_state;
    p.ck = (uint8_t*)d_cache_k; p.cv = (uint8_t*)d_cache_v; p.valid = d_valid;
    p.N = n_tokens; p.Nc = cdiv(n_tokens, C); p.n_full = n_tokens / C; p.C = C; p.SW = SW; p.Lcap = Lcap; p.rowB = D * 2;
    p.nB = cdiv(SW, kTokPerBlock);
    const int nC = cdiv(Lcap - SW, kTokPerBlock);
    dim3 grid(p.nB + nC, B * Hkv);
    evict_compact_kernel<<<grid, kCopyThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_cache_append(
    const void* d_k_new, const void* d_v_new, void* d_cache_k, void* d_cache_v, uint8_t* d_valid,
    int B, int Hkv, int x_len, int D, int Lcap, int pos, void* stream) {
    NATS_CHECK_ARG(B > 0 && Hkv > 0 && x_len > 0 && (long long)B * Hkv <= 65535, "bad shape B=%d Hkv=%d x_len=%d", B, Hkv, x_len);
    if (int rc = check_row(D)) return rc;
    NATS_CHECK_ARG(d_k_new && d_v_new && d_cache_k && d_cache_v && d_valid, "null pointer");
    NATS_CHECK_ARG(((uintptr_t)d_k_new | (uintptr_t)d_v_new | (uintptr_t)d_cache_k | (uintptr_t)d_cache_v) % 16 == 0,
                   "K/V and cache pointers must be 16-byte aligned");
    NATS_CHECK_ARG(pos >= 0 && (long long)pos + x_len <= Lcap, "rows [%d, %d) do not fit the cache capacity %d", pos, pos + x_len, Lcap);
    AppendParams p;
    p.k = (const uint8_t*)d_k_new; p.v = (const uint8_t*)d_v_new;
    p.ck = (uint8_t*)d_cache_k; p.cv = (uint8_t*)d_cache_v; p.valid = d_valid;
    p.x_len = x_len; p.pos = pos; p.Lcap = Lcap; p.rowB = D * 2;
    dim3 grid(cdiv(x_len, kTokPerBlock), B * Hkv);
    cache_append_kernel<<<grid, kCopyThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

// One thread: the step counters of the static decode step.  state[4] = tokens in the unfinished chunk, state[5] = ring
// write position.  Runs behind the (conditional) placement kernel of the same step.
__global__ void decode_step_advance_kernel(int32_t* state, int C, int SW) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const int fill = state[4] + 1;
    if (fill == C) {
        state[4] = 0;
        state[5] = (state[5] + C) % SW;
    } else {
        state[4] = fill;
    }
}

extern "C" __attribute__((visibility("default"))) int nats_b200_decode_step_place(const uint8_t* d_roles, void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                                                                       int64_t* d_size_global, int64_t* d_size_local, int32_t* d_state,
                                                                       int B, int Hkv, int D, int C, int SW, void* stream) {
    if (int rc = check_common(B, Hkv, 1, C, SW)) return rc;
    if (int rc = check_row(D)) return rc;
    NATS_CHECK_ARG(d_roles && d_cache_k && d_cache_v && d_valid && d_size_global && d_size_local && d_state, "null pointer");
    PlaceParams p;
    p.roles = d_roles; p.ck = (uint8_t*)d_cache_k; p.cv = (uint8_t*)d_cache_v; p.valid = d_valid;
    p.size_global = (long long*)d_size_global; p.size_local = (long long*)d_size_local; p.state = d_state;
    p.C = C; p.SW = SW; p.Lcap = Lcap; p.rowB = D * 2; p.tail = 0; p.from_state = 1;
    decode_place_kernel<<<B * Hkv, kCopyThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    decode_step_advance_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(d_state, C, SW);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}

extern "C" __attribute__((visibility("default"))) int nats_b200_decode_place(const uint8_t* d_roles, void* d_cache_k, void* d_cache_v, uint8_t* d_valid, int Lcap,
                                      int64_t* d_size_global, int64_t* d_size_local, int32_t* d_state,
                                      int tail, int B, int Hkv, int D, int C, int SW, void* stream) {
    if (int rc = check_common(B, Hkv, 1, C, SW)) return rc;
    if (int rc = check_row(D)) return rc;
    NATS_CHECK_ARG(d_roles && d_cache_k && d_cache_v && d_valid && d_size_global && d_size_local && d_state, "null pointer");
    NATS_CHECK_ARG(tail >= 0 && tail < SW && tail % C == 0, "ring tail %d must be a chunk multiple inside the window %d", tail, SW);
    PlaceParams p;
    p.roles = d_roles; p.ck = (uint8_t*)d_cache_k; p.cv = (uint8_t*)d_cache_v; p.valid = d_valid;
    p.size_global = (long long*)d_size_global; p.size_local = (long long*)d_size_local; p.state = d_state;
    p.C = C; p.SW = SW; p.Lcap = Lcap; p.rowB = D * 2; p.tail = tail; p.from_state = 0;
    decode_place_kernel<<<B * Hkv, kCopyThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}
