// Rotary position embedding fused with the head split: reads the q / k / v projections as the linear layers leave them
// ([B, N, H*D], one row per token) and writes [B, H, N, D] tensors, q and k rotated.  HBM-bound: every element is read
// once and written once with 16-byte accesses (the unfused chain -- two multiplies, a half rotation, an add and a
// .contiguous() per tensor -- moves the same data four to five times).
//
// The arithmetic reproduces the bf16 element-wise chain of the callers it replaces bit for bit:
// out = bf16(bf16(x * cos) + bf16(rotate_half(x) * sin)), each product and the sum rounded to bf16 (round to nearest even).
#include "common.cuh"

namespace nats {

struct RopeParams {
    const __nv_bfloat16* q_in; const __nv_bfloat16* k_in; const __nv_bfloat16* v_in;
    long long sq, sk, sv;                 // elements between consecutive tokens of the inputs
    const __nv_bfloat16* cos; const __nv_bfloat16* sin;
    long long cs_batch;                   // elements between batches of cos / sin (0: shared by the batch)
    __nv_bfloat16* q_out; __nv_bfloat16* k_out; __nv_bfloat16* v_out;
    int B, N, Hq, Hkv, D;
};

constexpr int kRopeThreads = 256;
constexpr int kRopeTokens = 8;            // tokens per block

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// 8 bf16 values in a uint4
struct Vec8 { float f[8]; };
__device__ __forceinline__ Vec8 unpack8(uint4 u) {
    Vec8 r;
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r.f[2 * i] = __uint_as_float(w[i] << 16);
        r.f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
    return r;
}
__device__ __forceinline__ uint4 pack8(const Vec8& v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(v.f[2 * i], v.f[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void __launch_bounds__(kRopeThreads) rope_split_heads_kernel(const RopeParams p) {
    const int b = blockIdx.y;
    const int t0 = blockIdx.x * kRopeTokens;
    const int vph = p.D / 16;                           // 16-byte vectors per half head
    const int Ht = p.Hq + 2 * p.Hkv;
    const int units = kRopeTokens * Ht * vph;
    for (int u = threadIdx.x; u < units; u += kRopeThreads) {
        const int j = u % vph;
        const int h = (u / vph) % Ht;
        const int t = t0 + u / (vph * Ht);
        if (t >= p.N) break;
        const __nv_bfloat16* in;
        __nv_bfloat16* out;
        bool rotate = true;
        if (h < p.Hq) {
            in = p.q_in + ((size_t)b * p.N + t) * p.sq + (size_t)h * p.D;
            out = p.q_out + (((size_t)b * p.Hq + h) * p.N + t) * p.D;
        } else if (h < p.Hq + p.Hkv) {
            const int hk = h - p.Hq;
            in = p.k_in + ((size_t)b * p.N + t) * p.sk + (size_t)hk * p.D;
            out = p.k_out + (((size_t)b * p.Hkv + hk) * p.N + t) * p.D;
        } else {
            const int hv = h - p.Hq - p.Hkv;
            in = p.v_in + ((size_t)b * p.N + t) * p.sv + (size_t)hv * p.D;
            out = p.v_out + (((size_t)b * p.Hkv + hv) * p.N + t) * p.D;
            rotate = false;
        }
        const int lo = j * 8, hi = p.D / 2 + j * 8;
        const uint4 r1 = ld16_stream(in + lo), r2 = ld16_stream(in + hi);
        if (!rotate) {
            st16(out + lo, r1);
            st16(out + hi, r2);
            continue;
        }
        const __nv_bfloat16* cs = p.cos + (size_t)b * p.cs_batch + (size_t)t * p.D;
        const __nv_bfloat16* sn = p.sin + (size_t)b * p.cs_batch + (size_t)t * p.D;
        const Vec8 x1 = unpack8(r1), x2 = unpack8(r2);
        const Vec8 c1 = unpack8(ld16(cs + lo)), c2 = unpack8(ld16(cs + hi));
        const Vec8 s1 = unpack8(ld16(sn + lo)), s2 = unpack8(ld16(sn + hi));
        Vec8 o1, o2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // first half: x1 * cos - x2 * sin; second half: x2 * cos + x1 * sin (rotate_half = [-x2, x1])
            o1.f[i] = bf16_round(__fmul_rn(x1.f[i], c1.f[i])) + bf16_round(__fmul_rn(-x2.f[i], s1.f[i]));
            o2.f[i] = bf16_round(__fmul_rn(x2.f[i], c2.f[i])) + bf16_round(__fmul_rn(x1.f[i], s2.f[i]));
        }
        st16(out + lo, pack8(o1));
        st16(out + hi, pack8(o2));
    }
}

}  // namespace nats

using namespace nats;

extern "C" __attribute__((visibility("default"))) int nats_b200_rope_split_heads(
    const void* d_q_in, const void* d_k_in, const void* d_v_in, long long q_token_stride, long long k_token_stride,
    long long v_token_stride, const void* d_cos, const void* d_sin, long long cos_batch_stride,
    void* d_q_out, void* d_k_out, void* d_v_out, int B, int N, int Hq, int Hkv, int D, void* stream) {
    NATS_CHECK_ARG(B > 0 && N > 0 && Hq > 0 && Hkv > 0 && B <= 65535, "bad shape B=%d N=%d Hq=%d Hkv=%d", B, N, Hq, Hkv);
    NATS_CHECK_ARG(D >= 16 && D % 16 == 0 && D <= 512, "head_dim %d must be a multiple of 16 up to 512", D);
    NATS_CHECK_ARG(d_q_in && d_k_in && d_v_in && d_cos && d_sin && d_q_out && d_k_out && d_v_out, "null pointer");
    NATS_CHECK_ARG(((uintptr_t)d_q_in | (uintptr_t)d_k_in | (uintptr_t)d_v_in | (uintptr_t)d_cos | (uintptr_t)d_sin |
                    (uintptr_t)d_q_out | (uintptr_t)d_k_out | (uintptr_t)d_v_out) % 16 == 0, "pointers must be 16-byte aligned");
    NATS_CHECK_ARG(q_token_stride >= (long long)Hq * D && k_token_stride >= (long long)Hkv * D && v_token_stride >= (long long)Hkv * D &&
                   q_token_stride % 8 == 0 && k_token_stride % 8 == 0 && v_token_stride % 8 == 0,
                   "token strides must cover a row of heads and keep 16-byte alignment");
    NATS_CHECK_ARG(cos_batch_stride == 0 || cos_batch_stride >= (long long)N * D, "bad cos/sin batch stride");
    RopeParams p;
    p.q_in = (const __nv_bfloat16*)d_q_in; p.k_in = (const __nv_bfloat16*)d_k_in; p.v_in = (const __nv_bfloat16*)d_v_in;
    p.sq = q_token_stride; p.sk = k_token_stride; p.sv = v_token_stride;
    p.cos = (const __nv_bfloat16*)d_cos; p.sin = (const __nv_bfloat16*)d_sin; p.cs_batch = cos_batch_stride;
    p.q_out = (__nv_bfloat16*)d_q_out; p.k_out = (__nv_bfloat16*)d_k_out; p.v_out = (__nv_bfloat16*)d_v_out;
    p.B = B; p.N = N; p.Hq = Hq; p.Hkv = Hkv; p.D = D;
    dim3 grid(cdiv(N, kRopeTokens), B);
    rope_split_heads_kernel<<<grid, kRopeThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}
