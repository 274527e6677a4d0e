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

constexpr int PREP_WARPS = 4;

template <typename OT>
__global__ void __launch_bounds__(PREP_WARPS * 32)
heads_prepare_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ pos,
                     const int* __restrict__ seq_of_token, const float* __restrict__ q_norm,
                     const float* __restrict__ k_norm, float eps, const float* __restrict__ freq, int rot,
                     float mscale, int num_tokens, int nh, int nkv, int d, int dv, int D, OT* __restrict__ q,
                     OT* __restrict__ k, OT* __restrict__ v, const PrepCommit c, int* status) {
    extern __shared__ float prep_buf[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int dmax = d > dv ? d : dv;
    float* buf = prep_buf + (size_t)warp * dmax;
    const int hs_count = nh + 2 * nkv;
    const long long row = (long long)blockIdx.x * PREP_WARPS + warp;
    pdl_sync();
    if (row >= (long long)num_tokens * hs_count) return;
    const int t = (int)(row / hs_count), hs = (int)(row % hs_count);
    const bool is_q = hs < nh, is_k = !is_q && hs < nh + nkv;
    const int head = is_q ? hs : is_k ? hs - nh : hs - nh - nkv;
    const int n = (is_q || is_k) ? d : dv;
    const float* src = proj + (size_t)t * ld + (is_q ? (size_t)head * d
                                                      : is_k ? (size_t)nh * d + (size_t)head * d
                                                             : (size_t)(nh + nkv) * d + (size_t)head * dv);
    const int p_int = pos[t];
    float ss = 0.f;
    for (int e = lane; e < n; e += 32) {
        const float x = src[e];
        buf[e] = x;
        ss += x * x;
    }
    const float* nw = is_q ? q_norm : is_k ? k_norm : nullptr;
    if (nw) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int e = lane; e < n; e += 32) buf[e] = buf[e] * inv * nw[e];
    }
    __syncwarp();
    if ((is_q || is_k) && rot > 0) {
        const int half = rot / 2;
        const float p = (float)p_int;
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf(p * freq[i], &sn, &cs);
            cs *= mscale, sn *= mscale;
            const float a = buf[i], b = buf[i + half];
            buf[i] = rot_lo(a, b, cs, sn);
            buf[i + half] = rot_hi(a, b, cs, sn);
        }
        __syncwarp();
    }
    OT* dst = is_q ? q + ((size_t)t * nh + head) * D : (is_k ? k : v) + ((size_t)t * nkv + head) * D;
    for (int e = lane; e < D; e += 32) st_f(dst + e, e < n ? buf[e] : 0.f);
    if (!is_q && c.k_cache) {
        const int s = seq_of_token[t];
        if (s >= 0 && !(c.ring > 0 && p_int < c.seq_end[s] - c.ring)) {
            const CachePos cp = cache_pos(p_int, c.ring, c.tables + (size_t)c.slots[s] * c.table_stride, c.page_size,
                                          c.num_pages, status);
            OT* cd = (OT*)(is_k ? c.k_cache : c.v_cache) + cache_index(cp, head, nkv, c.page_size, D);
            for (int e = lane; e < D; e += 32) st_f(cd + e, e < n ? buf[e] : 0.f);
        }
    }
}

// proj: [T, ld] 32-bit, bias added: q heads (nh * d), k heads (nkv * d), v heads (nkv * dv), then
// whatever else the layer projected.  q: [T, nh, D]; k, v: [T, nkv, D].
MOE_API int moe_heads_prepare(const float* proj, int ld, const int* pos, const int* seq_of_token, const float* q_norm,
                              const float* k_norm, float eps, const float* freq, int rot, float mscale,
                              int num_tokens, int nh, int nkv, int d, int dv, int D, void* q, void* k, void* v,
                              int out_dt, void* k_cache, void* v_cache, const int* seq_end, const int* slots,
                              const int* tables, int table_stride, int ring, int page_size, int num_pages,
                              int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && !freq) || d <= 0 || dv <= 0 || D < d || D < dv || !q ||
        !k || !v || ld < (nh + nkv) * d + nkv * dv)
        return (int)cudaErrorInvalidValue;
    if (k_cache && (!v_cache || !seq_end || !slots || !tables || !seq_of_token)) return (int)cudaErrorInvalidValue;
    PrepCommit c{k_cache, v_cache, seq_end, slots, tables, table_stride, ring, page_size, num_pages};
    const long long rows = (long long)num_tokens * (nh + 2 * nkv);
    const unsigned blocks = (unsigned)((rows + PREP_WARPS - 1) / PREP_WARPS);
    const size_t smem = (size_t)PREP_WARPS * (d > dv ? d : dv) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (out_dt == DT_F32)
        return launch_pdl(heads_prepare_kernel<float>, blocks, PREP_WARPS * 32, smem, stream, proj, ld, pos,
                          seq_of_token, q_norm, k_norm, eps, freq, rot, mscale, num_tokens, nh, nkv, d, dv, D,
                          (float*)q, (float*)k, (float*)v, c, status);
    return launch_pdl(heads_prepare_kernel<__nv_bfloat16>, blocks, PREP_WARPS * 32, smem, stream, proj, ld, pos,
                      seq_of_token, q_norm, k_norm, eps, freq, rot, mscale, num_tokens, nh, nkv, d, dv, D,
                      (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, c, status);
}

template <typename OT>
__global__ void gate_pack_kernel(const OT* __restrict__ ctx, const float* __restrict__ gate, int ld, long long total,
                                 int nh, int dv, int D, OT* __restrict__ out) {
    pdl_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int w = nh * dv;
    const long long t = i / w;
    const int c = (int)(i % w), h = c / dv, j = c % dv;
    float x = ld_f(ctx + ((size_t)t * nh + h) * D + j);
    if (gate) x *= 1.0f / (1.0f + expf(-gate[(size_t)t * ld + c]));
    st_f(out + i, x);
}

// ctx: [T, nh, D]; gate: first gate logit of token 0 (row pitch ld, 32-bit) or null; out: [T, nh * dv].
MOE_API int moe_gate_pack(const void* ctx, const float* gate, int ld, int num_tokens, int nh, int dv, int D, void* out,
                          int dt, cudaStream_t stream) {
    const long long total = (long long)num_tokens * nh * dv;
    if (total <= 0) return 0;
    if (D < dv) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dt == DT_F32)
        return launch_pdl(gate_pack_kernel<float>, blocks, 256, 0, stream, (const float*)ctx, gate, ld, total, nh, dv,
                          D, (float*)out);
    return launch_pdl(gate_pack_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)ctx, gate, ld,
                      total, nh, dv, D, (__nv_bfloat16*)out);
}
