// What lies between an attention layer's projection and its attention, and between the attention
// and the output projection, for layers whose heads need more than a rotation:
//
//   heads_prepare   per head of a token's 32-bit projection row [q heads | k heads | v heads | ...]:
//                   an optional RMS norm over the head (x / sqrt(mean(x^2) + eps) * w, one weight
//                   vector shared by the query heads and one by the key heads), then the rotation of
//                   the first `rot` dimensions (pairs (i, i + rot/2)) by angle pos * freq[i] with cos
//                   and sin multiplied by `mscale` (1 without context extension), then the split into
//                   q, k and v rows of the cache's record width D >= max(d, dv), zero-filled beyond
//                   the head's own width, so that query/key size and value size may differ: zeros
//                   add nothing to a score and give output columns that the next kernel drops.
//                   Optionally the keys and values are appended to the paged cache in the same
//                   launch (whole prompts and single-token steps).
//   gate_pack       out[t, h * dv + j] = ctx[t, h, j] * sigmoid(gate[t, h * dv + j]) (gate logits
//                   are columns of the same projection row; null: no gate), which also drops the
//                   padding columns.
// Norm, angles, rotation and the gate are 32-bit; only the stores round to the activation dtype.
#include "common.cuh"

struct PrepCommit {
    void* k_cache;            // null: no append
    void* v_cache;
    const int* seq_end;
    const int* slots;
    const int* tables;
    int table_stride, ring, page_size, num_pages;
};

constexpr int PREP_WARPS = 8;

__device__ __forceinline__ void prep_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void prep_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

// A block works on one token (grid.y == 1: many tokens, every warp takes heads in turn) or on
// PREP_WARPS heads of one token (few tokens: a warp a head, so that a step of one sequence is not one
// block).  The token's angles once a block (cos and sin of pos * freq[i], times mscale) in shared
// memory, then per head: load (four elements a lane where the sizes allow, VEC), sum of squares
// over the warp, scale, rotate through a per-warp buffer, store.
template <typename OT, bool VEC>
__global__ void __launch_bounds__(PREP_WARPS * 32)
heads_prepare_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ pos,
                     const int* __restrict__ seq_of_token, const float* __restrict__ q_norm,
                     const float* __restrict__ k_norm, float eps, const float* __restrict__ freq, int rot,
                     float mscale, int num_tokens, int nh, int nkv, int d, int dv, int D, OT* __restrict__ q,
                     OT* __restrict__ k, OT* __restrict__ v, long long ldq, long long ldkv, const PrepCommit c,
                     int* status) {
    extern __shared__ __align__(16) float prep_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int dmax = ((d > dv ? d : dv) + 3) & ~3;
    const int half = rot / 2;
    float* ang = prep_smem;                                    // cos[half], sin[half]
    float* buf = prep_smem + ((rot + 3) & ~3) + (size_t)warp * dmax;
    const int t = blockIdx.x;
    pdl_sync();
    const int p_int = pos[t];
    {
        const float p = (float)p_int;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf(p * freq[i], &sn, &cs);
            ang[i] = cs * mscale, ang[half + i] = sn * mscale;
        }
    }
    __syncthreads();
    // where the token's key and value go in the cache, if they are to be appended here
    bool append = false;
    CachePos cp;
    cp.page = 0, cp.off = 0;
    if (c.k_cache) {
        const int s = seq_of_token[t];
        if (s >= 0 && !(c.ring > 0 && p_int < c.seq_end[s] - c.ring)) {
            cp = cache_pos(p_int, c.ring, c.tables + (size_t)c.slots[s] * c.table_stride, c.page_size, c.num_pages,
                           status);
            append = true;
        }
    }
    const int hs_count = nh + 2 * nkv;
    const int step = gridDim.y * PREP_WARPS;
    const float* row = proj + (size_t)t * ld;
    // where head slot hs starts in the projection row
    auto head_src = [&](int hs) {
        return row + (hs < nh ? (size_t)hs * d
                              : hs < nh + nkv ? (size_t)nh * d + (size_t)(hs - nh) * d
                                              : (size_t)(nh + nkv) * d + (size_t)(hs - nh - nkv) * dv);
    };
    int hs = blockIdx.y * PREP_WARPS + warp;
    const bool in_regs = VEC && d <= 128 && dv <= 128 && D <= 128 && rot % 8 == 0;
    // (VEC) the first four elements a lane of the NEXT head are asked for before this head is worked
    // on, so that a warp has two loads in flight instead of one
    float4 ahead = make_float4(0.f, 0.f, 0.f, 0.f);
    if (VEC && hs < hs_count && lane * 4 < (hs < nh + nkv ? d : dv))
        ahead = *reinterpret_cast<const float4*>(head_src(hs) + lane * 4);
    for (; hs < hs_count; hs += step) {
        const bool is_q = hs < nh, is_k = !is_q && hs < nh + nkv;
        const int head = is_q ? hs : is_k ? hs - nh : hs - nh - nkv;
        const int n = (is_q || is_k) ? d : dv;
        const float* src = head_src(hs);
        float ss = 0.f;
        float4 first = ahead;
        if (VEC) {
            const int nx = hs + step;
            if (nx < hs_count && lane * 4 < (nx < nh + nkv ? d : dv))
                ahead = *reinterpret_cast<const float4*>(head_src(nx) + lane * 4);
        }
        OT* dst = is_q ? q + (size_t)t * ldq + (size_t)head * D : (is_k ? k : v) + (size_t)t * ldkv + (size_t)head * D;
        OT* cd = (!is_q && append) ? (OT*)(is_k ? c.k_cache : c.v_cache) + cache_index(cp, head, nkv, c.page_size, D)
                                   : nullptr;
        if (VEC && in_regs) {
            // heads of up to 128 with a rotated width that is a multiple of 8: a lane keeps its four
            // elements in registers throughout, and the rotation's partner (i <-> i + rot/2) is the
            // lane rot/8 further on or back
            const bool mine = lane * 4 < n;
            float4 x = mine ? first : make_float4(0.f, 0.f, 0.f, 0.f);
            const float* nw = is_q ? q_norm : is_k ? k_norm : nullptr;
            if (nw) {
                ss = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
                const float inv = 1.0f / sqrtf(ss / (float)d + eps);
                if (mine) {
                    const float4 w = *reinterpret_cast<const float4*>(nw + lane * 4);
                    x.x = x.x * inv * w.x, x.y = x.y * inv * w.y, x.z = x.z * inv * w.z, x.w = x.w * inv * w.w;
                }
            }
            if ((is_q || is_k) && rot > 0) {
                const int hl = half / 4;                   // lanes that hold one half of the rotated part
                const int from = lane < hl ? lane + hl : lane < 2 * hl ? lane - hl : lane;
                float4 y;
                y.x = __shfl_sync(0xffffffffu, x.x, from), y.y = __shfl_sync(0xffffffffu, x.y, from);
                y.z = __shfl_sync(0xffffffffu, x.z, from), y.w = __shfl_sync(0xffffffffu, x.w, from);
                if (lane < 2 * hl) {
                    const int i0 = (lane < hl ? lane : lane - hl) * 4;
                    const float4 cs = *reinterpret_cast<const float4*>(ang + i0);
                    const float4 sn = *reinterpret_cast<const float4*>(ang + half + i0);
                    if (lane < hl) {
                        x.x = rot_lo(x.x, y.x, cs.x, sn.x), x.y = rot_lo(x.y, y.y, cs.y, sn.y);
                        x.z = rot_lo(x.z, y.z, cs.z, sn.z), x.w = rot_lo(x.w, y.w, cs.w, sn.w);
                    } else {
                        x.x = rot_hi(y.x, x.x, cs.x, sn.x), x.y = rot_hi(y.y, x.y, cs.y, sn.y);
                        x.z = rot_hi(y.z, x.z, cs.z, sn.z), x.w = rot_hi(y.w, x.w, cs.w, sn.w);
                    }
                }
            }
            if (lane * 4 < D) {
                prep_store4(dst + lane * 4, x.x, x.y, x.z, x.w);
                if (cd) prep_store4(cd + lane * 4, x.x, x.y, x.z, x.w);
            }
            continue;
        }
        if (VEC) {
            for (int e = lane * 4; e < n; e += 128) {
                const float4 x = e < 128 ? first : *reinterpret_cast<const float4*>(src + e);
                *reinterpret_cast<float4*>(buf + e) = x;
                ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
            }
        } else {
            for (int e = lane; e < n; e += 32) {
                const float x = src[e];
                buf[e] = x;
                ss += x * x;
            }
        }
        const float* nw = is_q ? q_norm : is_k ? k_norm : nullptr;
        if (nw) {
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)d + eps);
            // (each lane scales the elements it loaded itself)
            if (VEC) {
                for (int e = lane * 4; e < n; e += 128) {
                    float4 x = *reinterpret_cast<float4*>(buf + e);
                    const float4 w = *reinterpret_cast<const float4*>(nw + e);
                    x.x = x.x * inv * w.x, x.y = x.y * inv * w.y, x.z = x.z * inv * w.z, x.w = x.w * inv * w.w;
                    *reinterpret_cast<float4*>(buf + e) = x;
                }
            } else {
                for (int e = lane; e < n; e += 32) buf[e] = buf[e] * inv * nw[e];
            }
        }
        __syncwarp();
        if ((is_q || is_k) && rot > 0) {
            for (int i = lane; i < half; i += 32) {
                const float cs = ang[i], sn = ang[half + i];
                const float a = buf[i], b = buf[i + half];
                buf[i] = rot_lo(a, b, cs, sn);
                buf[i + half] = rot_hi(a, b, cs, sn);
            }
            __syncwarp();
        }
        if (VEC) {
            for (int e = lane * 4; e < D; e += 128) {
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e < n) x = *reinterpret_cast<const float4*>(buf + e);
                prep_store4(dst + e, x.x, x.y, x.z, x.w);
                if (cd) prep_store4(cd + e, x.x, x.y, x.z, x.w);
            }
        } else {
            for (int e = lane; e < D; e += 32) {
                const float x = e < n ? buf[e] : 0.f;
                st_f(dst + e, x);
                if (cd) st_f(cd + e, x);
            }
        }
        __syncwarp();
    }
}

// proj: [T, ld] 32-bit, bias added: q heads (nh * d), k heads (nkv * d), v heads (nkv * dv), then
// whatever else the layer projected.  q: [T, nh, D] with a token pitch of ldq elements; k, v:
// [T, nkv, D] with a token pitch of ldkv (so the three may be parts of one row [q | k | v]).
MOE_API int moe_heads_prepare(const float* proj, int ld, const int* pos, const int* seq_of_token, const float* q_norm,
                              const float* k_norm, float eps, const float* freq, int rot, float mscale,
                              int num_tokens, int nh, int nkv, int d, int dv, int D, void* q, void* k, void* v,
                              long long ldq, long long ldkv, int out_dt, void* k_cache, void* v_cache, const int* seq_end, const int* slots,
                              const int* tables, int table_stride, int ring, int page_size, int num_pages,
                              int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && !freq) || d <= 0 || dv <= 0 || D < d || D < dv || !q ||
        !k || !v || ld < (nh + nkv) * d + nkv * dv || ldq < (long long)nh * D || ldkv < (long long)nkv * D)
        return (int)cudaErrorInvalidValue;
    if (k_cache && (!v_cache || !seq_end || !slots || !tables || !seq_of_token)) return (int)cudaErrorInvalidValue;
    PrepCommit c{k_cache, v_cache, seq_end, slots, tables, table_stride, ring, page_size, num_pages};
    const int dmax = ((d > dv ? d : dv) + 3) & ~3;
    const size_t smem = ((size_t)((rot + 3) & ~3) + (size_t)PREP_WARPS * dmax) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    // few tokens: a warp per head; from 128 tokens on the blocks fill the GPU anyway and a block per
    // token forms the token's angles once
    const dim3 grid(num_tokens, num_tokens >= 128 ? 1 : (nh + 2 * nkv + PREP_WARPS - 1) / PREP_WARPS);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    const size_t esz = out_dt == DT_F32 ? 4 : 2;
    auto al = [](const void* p, size_t a) { return ((uintptr_t)p % a) == 0; };
    const bool vec = d % 4 == 0 && dv % 4 == 0 && D % 4 == 0 && ld % 4 == 0 && ldq % 4 == 0 && ldkv % 4 == 0 &&
                     al(proj, 16) && al(q_norm, 16) && al(k_norm, 16) && al(q, 4 * esz) && al(k, 4 * esz) &&
                     al(v, 4 * esz) && al(k_cache, 4 * esz) && al(v_cache, 4 * esz);
#define PREP(OT_, VEC_)                                                                                             \
    return launch_pdl(heads_prepare_kernel<OT_, VEC_>, grid, PREP_WARPS * 32, smem, stream, proj, ld, pos,          \
                      seq_of_token, q_norm, k_norm, eps, freq, rot, mscale, num_tokens, nh, nkv, d, dv, D, (OT_*)q, \
                      (OT_*)k, (OT_*)v, ldq, ldkv, c, status)
    if (out_dt == DT_F32) {
        if (vec) PREP(float, true);
        PREP(float, false);
    }
    if (vec) PREP(__nv_bfloat16, true);
    PREP(__nv_bfloat16, false);
#undef PREP
}

__device__ __forceinline__ float4 prep_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 prep_load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ float sigmoid32(float x) { return 1.0f / (1.0f + expf(-x)); }

// One thread per four consecutive columns of a head (VEC) or per element.
template <typename OT, bool VEC>
__global__ void gate_pack_kernel(const OT* __restrict__ ctx, const float* __restrict__ gate, int ld, long long total,
                                 int nh, int dv, int D, OT* __restrict__ out) {
    pdl_sync();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
    if (i >= total) return;
    const int w = nh * dv;
    const long long t = i / w;
    const int c = (int)(i % w), h = c / dv, j = c % dv;
    if (VEC) {
        float4 x = prep_load4(ctx + ((size_t)t * nh + h) * D + j);
        if (gate) {
            const float4 g = *reinterpret_cast<const float4*>(gate + (size_t)t * ld + c);
            x.x *= sigmoid32(g.x), x.y *= sigmoid32(g.y), x.z *= sigmoid32(g.z), x.w *= sigmoid32(g.w);
        }
        prep_store4(out + i, x.x, x.y, x.z, x.w);
    } else {
        float x = ld_f(ctx + ((size_t)t * nh + h) * D + j);
        if (gate) x *= sigmoid32(gate[(size_t)t * ld + c]);
        st_f(out + i, x);
    }
}

// ctx: [T, nh, D]; gate: first gate logit of token 0 (row pitch ld, 32-bit) or null; out: [T, nh * dv].
MOE_API int moe_gate_pack(const void* ctx, const float* gate, int ld, int num_tokens, int nh, int dv, int D, void* out,
                          int dt, cudaStream_t stream) {
    const long long total = (long long)num_tokens * nh * dv;
    if (total <= 0) return 0;
    if (D < dv) return (int)cudaErrorInvalidValue;
    const size_t esz = dt == DT_F32 ? 4 : 2;
    const bool vec = dv % 4 == 0 && D % 4 == 0 && ld % 4 == 0 && ((uintptr_t)gate % 16) == 0 &&
                     ((uintptr_t)ctx % (4 * esz)) == 0 && ((uintptr_t)out % (4 * esz)) == 0;
    const long long threads = vec ? total / 4 : total;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
#define PACK(OT_, VEC_)                                                                                        \
    return launch_pdl(gate_pack_kernel<OT_, VEC_>, blocks, 256, 0, stream, (const OT_*)ctx, gate, ld, total, nh, dv, \
                      D, (OT_*)out)
    if (dt == DT_F32) {
        if (vec) PACK(float, true);
        PACK(float, false);
    }
    if (vec) PACK(__nv_bfloat16, true);
    PACK(__nv_bfloat16, false);
#undef PACK
}
