// Dynamic Tanh, a norm without statistics: y = tanh(alpha * x) * w + b, elementwise, with a scalar
// alpha and vectors w and b.  As the RMS norm kernel does, this one first adds what the sublayer
// before it left pending to the 32-bit residual stream, and where that sublayer's output goes
// through a Dynamic Tanh of its own before the sum (a block with norms after its sublayers), that
// one is formed here as well:
//     x   <- x + (post ? tanh(pa * delta) * pw + pb : delta)        (stored back on request)
//     out <- pre ? tanh(a * x) * w + b : x                          (32-bit and / or bfloat16)
// so a block with four such norms reads and writes the stream once per sublayer.  Everything is
// 32-bit; only the second output is rounded to bfloat16 for the matrix product that follows.  The
// outputs have a row pitch of their own, so a caller may fill one half of a wider buffer.
#include "common.cuh"

struct DytParams {
    const float* alpha;   // device scalar; null: this stage is the identity
    const float* w;
    const float* b;
};

__device__ __forceinline__ float dyt1(float v, float a, float w, float b) { return fmaf(tanhf(a * v), w, b); }

// One block per output row i; source row r = rows ? rows[i] : i.
template <bool VEC>
__global__ void __launch_bounds__(256)
dyt_kernel(float* __restrict__ x, const float* __restrict__ delta, const DytParams post, const DytParams pre,
           const int* __restrict__ rows, float* __restrict__ out32, __nv_bfloat16* __restrict__ out16, int ld_out,
           int S, int H, int write_back, int* status) {
    // the norms' constants do not depend on the kernel before this one
    const float pa = post.alpha ? *post.alpha : 0.f, a = pre.alpha ? *pre.alpha : 0.f;
    pdl_sync();
    const int i = blockIdx.x;
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= S) {
        if (threadIdx.x == 0 && status) atomicOr(status, ST_BAD_ROW);
        r = 0;
    }
    float* xr = x + (size_t)r * H;
    const float* dr = delta ? delta + (size_t)r * H : nullptr;
    float* o32 = out32 ? out32 + (size_t)i * ld_out : nullptr;
    __nv_bfloat16* o16 = out16 ? out16 + (size_t)i * ld_out : nullptr;
    if (VEC) {
        for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(xr + c);
            if (dr) {
                float4 d = *reinterpret_cast<const float4*>(dr + c);
                if (post.alpha) {
                    const float4 w = *reinterpret_cast<const float4*>(post.w + c);
                    const float4 b = *reinterpret_cast<const float4*>(post.b + c);
                    d.x = dyt1(d.x, pa, w.x, b.x), d.y = dyt1(d.y, pa, w.y, b.y);
                    d.z = dyt1(d.z, pa, w.z, b.z), d.w = dyt1(d.w, pa, w.w, b.w);
                }
                v.x += d.x, v.y += d.y, v.z += d.z, v.w += d.w;
                if (write_back) *reinterpret_cast<float4*>(xr + c) = v;
            }
            if (pre.alpha) {
                const float4 w = *reinterpret_cast<const float4*>(pre.w + c);
                const float4 b = *reinterpret_cast<const float4*>(pre.b + c);
                v.x = dyt1(v.x, a, w.x, b.x), v.y = dyt1(v.y, a, w.y, b.y);
                v.z = dyt1(v.z, a, w.z, b.z), v.w = dyt1(v.w, a, w.w, b.w);
            }
            if (o32) *reinterpret_cast<float4*>(o32 + c) = v;
            if (o16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                uint2 u;
                u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
                *reinterpret_cast<uint2*>(o16 + c) = u;
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = xr[c];
            if (dr) {
                float d = dr[c];
                if (post.alpha) d = dyt1(d, pa, post.w[c], post.b[c]);
                v += d;
                if (write_back) xr[c] = v;
            }
            if (pre.alpha) v = dyt1(v, a, pre.w[c], pre.b[c]);
            if (o32) o32[c] = v;
            if (o16) o16[c] = __float2bfloat16_rn(v);
        }
    }
}

static inline bool al16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// x: [S, H] 32-bit stream; delta: [S, H] or null; post_* / pre_*: the two norms (alpha null: identity);
// rows: n_out source rows or null (then n_out == S); out32 / out16: [n_out, ld_out], either may be null.
MOE_API int moe_dyt(float* x, const float* delta, const float* post_alpha, const float* post_w, const float* post_b,
                    const float* pre_alpha, const float* pre_w, const float* pre_b, const int* rows, float* out32,
                    void* out16, int ld_out, int n_out, int S, int H, int write_back, int* status,
                    cudaStream_t stream) {
    if (n_out <= 0 || H <= 0) return 0;
    if ((post_alpha && (!post_w || !post_b)) || (pre_alpha && (!pre_w || !pre_b)) || ld_out < H)
        return (int)cudaErrorInvalidValue;
    DytParams post{post_alpha, post_w, post_b}, pre{pre_alpha, pre_w, pre_b};
    const bool vec = H % 4 == 0 && ld_out % 4 == 0 && al16(x) && al16(delta) && al16(post_w) && al16(post_b) &&
                     al16(pre_w) && al16(pre_b) && al16(out32) && ((uintptr_t)out16 & 7) == 0;
    const int per = vec ? 4 : 1;
    int threads = (H / per + 31) / 32 * 32;
    threads = threads < 32 ? 32 : threads > 256 ? 256 : threads;
    if (vec)
        return launch_pdl(dyt_kernel<true>, n_out, threads, 0, stream, x, delta, post, pre, rows, out32,
                          (__nv_bfloat16*)out16, ld_out, S, H, write_back, status);
    return launch_pdl(dyt_kernel<false>, n_out, threads, 0, stream, x, delta, post, pre, rows, out32,
                      (__nv_bfloat16*)out16, ld_out, S, H, write_back, status);
}
