// Between an attention layer's projection and its attention, for layers whose queries, keys and
// values pass a short causal convolution over time:
//
//   conv_heads_prepare   per channel c of a token's 32-bit projection row [q heads | k heads | v heads]
//                        y_t[c] = sum_j w[j, c] * u_(t - taps + 1 + j)[c]     (taps >= 1; 1: y = w u)
//                        where u of an earlier position comes from the step's own rows if that
//                        position belongs to the step, else from the sequence's state (the last
//                        taps - 1 projected rows before the step), and is zero before position 0.
//                        Then per query and key head: the rotation of the first `rot` dimensions,
//                        pairs (2i, 2i + 1) by the angle pos * freq[i] (the interleaved layout), and,
//                        if asked for, the division by the head's root mean square
//                        x / sqrt(mean(x^2) + eps), which has no weight.  Queries, keys and values
//                        are written as records of the cache's width D >= max(d, dv), zero-filled
//                        (see attention_prepare.cu), and keys and values may be appended to the
//                        paged cache in the same launch.
//   conv_state_update    after it: the state becomes the last taps - 1 projected rows of every
//                        sequence of the step (rows of the step, or what the state held, moved up).
//                        A launch of its own because the blocks above read the old state.
// Convolution, angles, rotation and norm are 32-bit; only the stores round to the activation dtype.
#include "common.cuh"

namespace {

struct ConvCommit {
    void* k_cache;            // null: no append
    void* v_cache;
    const int* seq_end;
    const int* tables;
    int table_stride, ring, page_size, num_pages;
};

constexpr int CONV_WARPS = 8;
constexpr int MAX_TAPS = 16;

__device__ __forceinline__ void conv_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void conv_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

// VEC: a lane works on four neighbouring channels at a time and keeps them in registers from the
// convolution to the store (heads of up to 256); a pair (2i, 2i + 1) lies within a lane's four.
template <typename OT, bool VEC>
__global__ void __launch_bounds__(CONV_WARPS * 32)
conv_heads_prepare_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ taps_w, int taps,
                          const float* __restrict__ state, long long state_pitch, const int* __restrict__ pos,
                          const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                          const int* __restrict__ slots, float eps, int unit_norm, const float* __restrict__ freq,
                          int rot, int nh, int nkv, int d, int dv, int D, OT* __restrict__ q, OT* __restrict__ k,
                          OT* __restrict__ v, long long ldq, long long ldkv, const ConvCommit c, int* status) {
    extern __shared__ __align__(16) float conv_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int dmax = d > dv ? d : dv;
    const int half = rot / 2;
    float* ang = conv_smem;                                    // cos[half], sin[half]
    float* buf = conv_smem + rot + (size_t)warp * dmax;
    const int t = blockIdx.x;
    const int channels = (nh + nkv) * d + nkv * dv;
    pdl_sync();
    const int s = seq_of_token[t];
    const int p_int = s < 0 ? 0 : pos[t];
    {
        const float p = (float)p_int;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf(p * freq[i], &sn, &cs);
            ang[i] = cs, ang[half + i] = sn;
        }
    }
    __syncthreads();
    const int tok0 = s < 0 ? t : cu_seqlens[s];
    const int r_in_step = t - tok0;                            // the token's place among its sequence's rows
    const float* st = (s >= 0 && state) ? state + (size_t)slots[s] * state_pitch : nullptr;
    bool append = false;
    CachePos cp;
    cp.page = 0, cp.off = 0;
    if (c.k_cache && s >= 0 && !(c.ring > 0 && p_int < c.seq_end[s] - c.ring)) {
        cp = cache_pos(p_int, c.ring, c.tables + (size_t)slots[s] * c.table_stride, c.page_size, c.num_pages, status);
        append = true;
    }
    const int hs_count = nh + 2 * nkv;
    for (int hs = blockIdx.y * CONV_WARPS + warp; hs < hs_count; hs += gridDim.y * CONV_WARPS) {
        const bool is_q = hs < nh, is_k = !is_q && hs < nh + nkv;
        const int head = is_q ? hs : is_k ? hs - nh : hs - nh - nkv;
        const int n = (is_q || is_k) ? d : dv;
        const int ch0 = is_q ? hs * d : is_k ? nh * d + head * d : (nh + nkv) * d + head * dv;
        OT* dst = is_q ? q + (size_t)t * ldq + (size_t)head * D : (is_k ? k : v) + (size_t)t * ldkv + (size_t)head * D;
        OT* cd = (!is_q && append) ? (OT*)(is_k ? c.k_cache : c.v_cache) + cache_index(cp, head, nkv, c.page_size, D)
                                   : nullptr;
        if (s < 0) {                                           // a row of no sequence: zeros
            for (int e = lane; e < D; e += 32) st_f(dst + e, 0.f);
            continue;
        }
        if (VEC) {
            float4 x[2];
            float ss = 0.f;
#pragma unroll
            for (int it = 0; it < 2; it++) {
                const int e = lane * 4 + it * 128;
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e < n) {
                    const int ch = ch0 + e;
                    if (!taps_w) {
                        y = *reinterpret_cast<const float4*>(proj + (size_t)t * ld + ch);
                    } else {
                        for (int j = 0; j < taps; j++) {
                            const int back = taps - 1 - j;
                            if (p_int - back < 0) continue;
                            const int r = r_in_step - back;
                            const float4 u = *reinterpret_cast<const float4*>(
                                r >= 0 ? proj + (size_t)(tok0 + r) * ld + ch : st + (size_t)(taps - 1 + r) * channels + ch);
                            const float4 w = *reinterpret_cast<const float4*>(taps_w + (size_t)j * channels + ch);
                            y.x = fmaf(w.x, u.x, y.x), y.y = fmaf(w.y, u.y, y.y), y.z = fmaf(w.z, u.z, y.z), y.w = fmaf(w.w, u.w, y.w);
                        }
                    }
                    if ((is_q || is_k) && e < rot) {
                        const float2 cs = *reinterpret_cast<const float2*>(ang + e / 2);
                        const float2 sn = *reinterpret_cast<const float2*>(ang + half + e / 2);
                        const float a0 = y.x, b0 = y.y, a1 = y.z, b1 = y.w;
                        y.x = rot_lo(a0, b0, cs.x, sn.x), y.y = rot_hi(a0, b0, cs.x, sn.x);
                        y.z = rot_lo(a1, b1, cs.y, sn.y), y.w = rot_hi(a1, b1, cs.y, sn.y);
                    }
                    ss = fmaf(y.x, y.x, ss), ss = fmaf(y.y, y.y, ss), ss = fmaf(y.z, y.z, ss), ss = fmaf(y.w, y.w, ss);
                }
                x[it] = y;
            }
            float inv = 1.0f;
            if ((is_q || is_k) && unit_norm) inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
#pragma unroll
            for (int it = 0; it < 2; it++) {
                const int e = lane * 4 + it * 128;
                if (e < D) {
                    conv_store4(dst + e, x[it].x * inv, x[it].y * inv, x[it].z * inv, x[it].w * inv);
                    if (cd) conv_store4(cd + e, x[it].x * inv, x[it].y * inv, x[it].z * inv, x[it].w * inv);
                }
            }
            continue;
        }
        // ---- the convolution ------------------------------------------------------------------
        for (int e = lane; e < n; e += 32) {
            const int ch = ch0 + e;
            float y;
            if (!taps_w) {
                y = proj[(size_t)t * ld + ch];
            } else {
                y = 0.f;
                for (int j = 0; j < taps; j++) {
                    const int back = taps - 1 - j;
                    if (p_int - back < 0) continue;            // before the sequence's first token
                    const int r = r_in_step - back;
                    const float u = r >= 0 ? proj[(size_t)(tok0 + r) * ld + ch]
                                           : st[(size_t)(taps - 1 + r) * channels + ch];
                    y = fmaf(taps_w[(size_t)j * channels + ch], u, y);
                }
            }
            buf[e] = y;
        }
        __syncwarp();
        // ---- rotation of pairs (2i, 2i + 1) and the unit norm ----------------------------------
        if ((is_q || is_k) && rot > 0) {
            for (int i = lane; i < half; i += 32) {
                const float cs = ang[i], sn = ang[half + i];
                const float a = buf[2 * i], b = buf[2 * i + 1];
                buf[2 * i] = rot_lo(a, b, cs, sn);
                buf[2 * i + 1] = rot_hi(a, b, cs, sn);
            }
            __syncwarp();
        }
        float inv = 1.0f;
        if ((is_q || is_k) && unit_norm) {
            float ss = 0.f;
            for (int e = lane; e < n; e += 32) ss = fmaf(buf[e], buf[e], ss);
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)d + eps);
        }
        for (int e = lane; e < D; e += 32) {
            const float x = e < n ? buf[e] * inv : 0.f;
            st_f(dst + e, x);
            if (cd) st_f(cd + e, x);
        }
        __syncwarp();
    }
}

// One block per sequence of the step.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const float* __restrict__ proj, int ld, float* __restrict__ state, long long state_pitch,
                         int taps, int channels, const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
    pdl_sync();
    const int s = blockIdx.x;
    const int tok0 = cu_seqlens[s], cnt = cu_seqlens[s + 1] - tok0;
    if (cnt <= 0) return;                                      // a sequence of a padded step that brings nothing
    float* st = state + (size_t)slots[s] * state_pitch;
    for (int ch = threadIdx.x; ch < channels; ch += blockDim.x)
        for (int i = 0; i < taps - 1; i++) {                   // ascending: an entry is read before it is written
            const int r = cnt - (taps - 1) + i;
            st[(size_t)i * channels + ch] = r >= 0 ? proj[(size_t)(tok0 + r) * ld + ch]
                                                   : st[(size_t)(i + cnt) * channels + ch];
        }
}

}  // namespace

// proj: [T, ld] 32-bit, bias added: q heads (nh * d), k heads (nkv * d), v heads (nkv * dv).
// taps_w: [taps, channels] 32-bit (a tap's factors for all channels side by side) or null (no convolution); state: [slots + 1, state_pitch] 32-bit with
// (taps - 1) * channels floats used per slot (null if taps <= 1).  q: [T, nh, D] with a token pitch of
// ldq; k, v: [T, nkv, D] with a token pitch of ldkv.  freq: [rot / 2].
MOE_API int moe_conv_heads_prepare(const float* proj, int ld, const float* taps_w, int taps, const float* state,
                                   long long state_pitch, const int* pos, const int* seq_of_token,
                                   const int* cu_seqlens, const int* slots, float eps, int unit_norm, const float* freq,
                                   int rot, int num_tokens, int nh, int nkv, int d, int dv, int D, void* q, void* k,
                                   void* v, long long ldq, long long ldkv, int out_dt, void* k_cache, void* v_cache,
                                   const int* seq_end, const int* tables, int table_stride, int ring, int page_size,
                                   int num_pages, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    const int channels = (nh + nkv) * d + nkv * dv;
    if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && !freq) || d <= 0 || dv <= 0 || D < d || D < dv || !q || !k || !v ||
        ld < channels || ldq < (long long)nh * D || ldkv < (long long)nkv * D || !pos || !seq_of_token || !cu_seqlens ||
        !slots)
        return (int)cudaErrorInvalidValue;
    if (taps_w && (taps < 1 || taps > MAX_TAPS || (taps > 1 && (!state || state_pitch < (long long)(taps - 1) * channels))))
        return (int)cudaErrorInvalidValue;
    if (k_cache && (!v_cache || !seq_end || !tables)) return (int)cudaErrorInvalidValue;
    const ConvCommit c{k_cache, v_cache, seq_end, tables, table_stride, ring, page_size, num_pages};
    const int dmax = d > dv ? d : dv;
    const size_t smem = ((size_t)rot + (size_t)CONV_WARPS * dmax) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const dim3 grid(num_tokens, num_tokens >= 128 ? 1 : (nh + 2 * nkv + CONV_WARPS - 1) / CONV_WARPS);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    const size_t esz = out_dt == DT_F32 ? 4 : 2;
    auto al = [](const void* p, size_t a) { return ((uintptr_t)p % a) == 0; };
    const bool vec = d % 4 == 0 && dv % 4 == 0 && D % 4 == 0 && D <= 256 && rot % 4 == 0 && ld % 4 == 0 && ldq % 4 == 0 &&
                     ldkv % 4 == 0 && state_pitch % 4 == 0 && al(proj, 16) && al(taps_w, 16) && al(state, 16) &&
                     al(q, 4 * esz) && al(k, 4 * esz) && al(v, 4 * esz) && al(k_cache, 4 * esz) && al(v_cache, 4 * esz);
#define CONV(OT_, VEC_)                                                                                              \
    return launch_pdl(conv_heads_prepare_kernel<OT_, VEC_>, grid, CONV_WARPS * 32, smem, stream, proj, ld, taps_w, taps, \
                      state, state_pitch, pos, seq_of_token, cu_seqlens, slots, eps, unit_norm, freq, rot, nh, nkv, d,  \
                      dv, D, (OT_*)q, (OT_*)k, (OT_*)v, ldq, ldkv, c, status)
    if (out_dt == DT_F32) {
        if (vec) CONV(float, true);
        CONV(float, false);
    }
    if (vec) CONV(__nv_bfloat16, true);
    CONV(__nv_bfloat16, false);
#undef CONV
}

MOE_API int moe_conv_state_update(const float* proj, int ld, float* state, long long state_pitch, int taps,
                                  int channels, const int* cu_seqlens, const int* slots, int num_seqs,
                                  cudaStream_t stream) {
    if (num_seqs <= 0 || taps <= 1) return 0;
    if (!proj || !state || ld < channels || state_pitch < (long long)(taps - 1) * channels || taps > MAX_TAPS)
        return (int)cudaErrorInvalidValue;
    return launch_pdl(conv_state_update_kernel, dim3(num_seqs), 256, 0, stream, proj, ld, state, state_pitch, taps,
                      channels, cu_seqlens, slots);
}
