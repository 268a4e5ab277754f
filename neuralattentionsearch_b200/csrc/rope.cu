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

// bf16(a * b) for four packed pairs: the product of two bf16 values is exact in fp32, so one rounding either way
__device__ __forceinline__ uint4 mul8(uint4 a, uint4 b) {
    uint4 r;
    const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&b);
    __nv_bfloat162* z = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) z[i] = __hmul2(x[i], y[i]);
    return r;
}
__device__ __forceinline__ uint4 neg8(uint4 a) {
    return make_uint4(a.x ^ 0x80008000u, a.y ^ 0x80008000u, a.z ^ 0x80008000u, a.w ^ 0x80008000u);
}
// bf16(a + b), the sum taken in fp32 like the element-wise chain does
__device__ __forceinline__ uint4 add8(uint4 a, uint4 b) {
    const Vec8 x = unpack8(a), y = unpack8(b);
    Vec8 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.f[i] = __fadd_rn(x.f[i], y.f[i]);
    return pack8(o);
}

// VPH = 16-byte vectors per half head (D / 16), 0 = read it from the parameters
template <int VPH>
__global__ void __launch_bounds__(kRopeThreads) rope_split_heads_kernel(const RopeParams p) {
    const int b = blockIdx.y;
    const int t0 = blockIdx.x * kRopeTokens;
    const int vph = VPH > 0 ? VPH : p.D / 16;
    const int Ht = p.Hq + 2 * p.Hkv;
    // a thread keeps its vector index j; (token, head) pairs are walked without divisions
    const int j = threadIdx.x % vph;
    const int pair_stride = kRopeThreads / vph;          // host side guarantees that vph divides the block
    int h = threadIdx.x / vph, t = t0;
    while (h >= Ht) { h -= Ht; ++t; }
    const int t_end = min(t0 + kRopeTokens, p.N);
    const int lo = j * 8, hi = p.D / 2 + j * 8;
    while (t < t_end) {
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
        const uint4 x1 = ld16_stream(in + lo), x2 = ld16_stream(in + hi);
        if (!rotate) {
            st16(out + lo, x1);
            st16(out + hi, x2);
        } else {
            const __nv_bfloat16* cs = p.cos + (size_t)b * p.cs_batch + (size_t)t * p.D;
            const __nv_bfloat16* sn = p.sin + (size_t)b * p.cs_batch + (size_t)t * p.D;
            const uint4 c1 = ld16(cs + lo), c2 = ld16(cs + hi), s1 = ld16(sn + lo), s2 = ld16(sn + hi);
            // first half: x1 * cos - x2 * sin; second half: x2 * cos + x1 * sin (rotate_half = [-x2, x1])
            st16(out + lo, add8(mul8(x1, c1), mul8(neg8(x2), s1)));
            st16(out + hi, add8(mul8(x2, c2), mul8(x1, s2)));
        }
        h += pair_stride;
        while (h >= Ht) { h -= Ht; ++t; }
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
    NATS_CHECK_ARG(kRopeThreads % (D / 16) == 0, "head_dim %d: the vectors of a half head must divide the block of %d threads", D, kRopeThreads);
    if (D == 128) rope_split_heads_kernel<8><<<grid, kRopeThreads, 0, (cudaStream_t)stream>>>(p);
    else if (D == 64) rope_split_heads_kernel<4><<<grid, kRopeThreads, 0, (cudaStream_t)stream>>>(p);
    else rope_split_heads_kernel<0><<<grid, kRopeThreads, 0, (cudaStream_t)stream>>>(p);
    NATS_CHECK_CUDA(cudaGetLastError());
    return NATS_OK;
}
