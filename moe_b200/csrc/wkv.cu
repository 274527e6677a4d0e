// A recurrent mixer with a matrix-valued state per head and data-dependent decay (RWKV-style time
// mixing).  Three kernels around the projections:
//
//   wkv_shift_mix   every projection reads its own blend of the token's input n_t and the previous
//                   token's n_(t-1):  x_s = n_t + (n_(t-1) - n_t) * mu_s  for s of `streams` blends.
//                   The previous token of a step's first row is the sequence's state (zeros at
//                   position 0); the block of that row also stores the sequence's LAST row of the
//                   step as the new state (it alone reads the old one, element by element before it
//                   writes).  The last blend may go to a 32-bit buffer of its own (the decay's).
//   wkv_decay       w_t[i] = exp(-exp(w0[i] + sum_q W2[i][q] tanh(low_t[q]))), low = W1 x_w being the
//                   decay's first, narrow projection: the second projection, its bias and both
//                   exponentials in one pass, 32-bit.
//   wkv_scan        per (sequence, head), tokens in order:
//                       o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])
//                       S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
//                   S lives in 32-bit floats in the sequence's state and is
//                   held in registers over the step: a block owns SCAN_COLS value columns j of one
//                   head, eight lanes share a column (rows i = lane % 8 + 8 m), and the eight partial
//                   sums of o_t[j] are added by shuffles in a fixed order.  r, k and the decay of
//                   SCAN_TOK tokens at a time pass through shared memory.
//   wkv_finish      each head's o_t is divided by its root mean square (x / sqrt(mean(x^2) + eps)),
//                   multiplied by a weight per channel and by silu(gate projection), and rounded to
//                   the activation dtype for the output projection.
// Everything here is 32-bit arithmetic; only wkv_shift_mix and wkv_finish round their stores.
#include "common.cuh"

namespace {

constexpr int SCAN_COLS = 16, SCAN_KP = 8, SCAN_THREADS = SCAN_COLS * SCAN_KP, SCAN_TOK = 8;

template <typename OT>
__global__ void __launch_bounds__(256)
wkv_shift_mix_kernel(const float* __restrict__ h, const float* __restrict__ mu, int streams, float* __restrict__ state,
                     long long state_pitch, const int* __restrict__ seq_of_token, const int* __restrict__ pos,
                     const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int num_tokens, int width,
                     OT* __restrict__ out, float* __restrict__ last32) {
    pdl_sync();
    const int t = blockIdx.x;
    const int s = seq_of_token[t];
    const size_t plane = (size_t)num_tokens * width;
    if (s < 0) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            for (int m = 0; m < streams - (last32 ? 1 : 0); m++) st_f(out + m * plane + (size_t)t * width + c, 0.f);
            if (last32) last32[(size_t)t * width + c] = 0.f;
        }
        return;
    }
    const int tok0 = cu_seqlens[s], last = cu_seqlens[s + 1] - 1;
    const bool first = t == tok0;
    float* st = state + (size_t)slots[s] * state_pitch;
    const bool from_zero = pos[t] == 0;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float x = h[(size_t)t * width + c];
        float prev;
        if (first) {
            prev = from_zero ? 0.f : st[c];
            st[c] = h[(size_t)last * width + c];
        } else {
            prev = h[(size_t)(t - 1) * width + c];
        }
        const float diff = prev - x;
        for (int m = 0; m < streams; m++) {
            const float y = fmaf(diff, mu[(size_t)m * width + c], x);
            if (last32 && m == streams - 1)
                last32[(size_t)t * width + c] = y;
            else
                st_f(out + m * plane + (size_t)t * width + c, y);
        }
    }
}

constexpr int MAX_RANK = 256;
// One block per token: the token's narrow row through tanh into shared memory, then a thread a channel.
__global__ void __launch_bounds__(256)
wkv_decay_kernel(const float* __restrict__ low, const float* __restrict__ w2, const float* __restrict__ w0, int inner,
                 int rank, float* __restrict__ out) {
    __shared__ float th[MAX_RANK];
    pdl_sync();
    const int t = blockIdx.x;
    for (int q = threadIdx.x; q < rank; q += blockDim.x) th[q] = tanhf(low[(size_t)t * rank + q]);
    __syncthreads();
    for (int c = threadIdx.x; c < inner; c += blockDim.x) {
        float acc = 0.f;
        for (int q = 0; q < rank; q++) acc = fmaf(w2[(size_t)c * rank + q], th[q], acc);
        out[(size_t)t * inner + c] = expf(-expf(acc + w0[c]));
    }
}

template <int RPT>
__global__ void __launch_bounds__(SCAN_THREADS)
wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                const float* __restrict__ w, long long ld, const float* __restrict__ u, float* __restrict__ state, long long state_pitch, const int* __restrict__ cu_seqlens,
                const int* __restrict__ slots, int heads, int d, float* __restrict__ out) {
    extern __shared__ float scan_smem[];     // [SCAN_TOK][3][d]: r, k, decay
    pdl_sync();
    const int seq = blockIdx.z, head = blockIdx.y;
    const int tok0 = cu_seqlens[seq], cnt = cu_seqlens[seq + 1] - tok0;
    if (cnt <= 0) return;
    const int kp = threadIdx.x % SCAN_KP, col = blockIdx.x * SCAN_COLS + threadIdx.x / SCAN_KP;
    const bool live = col < d;
    const size_t hc = (size_t)head * d;
    float* S = state + (size_t)slots[seq] * state_pitch + hc * d;        // [d (i)][d (j)] of this head
    float sreg[RPT], ureg[RPT];
#pragma unroll
    for (int m = 0; m < RPT; m++) {
        const int i = kp + SCAN_KP * m;
        sreg[m] = (live && i < d) ? S[(size_t)i * d + col] : 0.f;
        ureg[m] = i < d ? u[hc + i] : 0.f;
    }
    for (int t0 = 0; t0 < cnt; t0 += SCAN_TOK) {
        const int nt = min(SCAN_TOK, cnt - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * d; idx += SCAN_THREADS) {
            const int tt = idx / d, i = idx % d;
            const size_t at = (size_t)(tok0 + t0 + tt) * ld + hc + i;
            float* row = scan_smem + (size_t)tt * 3 * d;
            row[i] = r[at];
            row[d + i] = k[at];
            row[2 * d + i] = w[at];
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float* row = scan_smem + (size_t)tt * 3 * d;
            const size_t tok = (size_t)(tok0 + t0 + tt);
            const float vj = live ? v[tok * ld + hc + col] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int m = 0; m < RPT; m++) {
                const int i = kp + SCAN_KP * m;
                if (i < d) {
                    const float kv = row[d + i] * vj;
                    acc = fmaf(row[i], fmaf(ureg[m], kv, sreg[m]), acc);
                    sreg[m] = fmaf(row[2 * d + i], sreg[m], kv);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (live && kp == 0) out[tok * ((size_t)heads * d) + hc + col] = acc;
        }
    }
    if (live)
#pragma unroll
        for (int m = 0; m < RPT; m++) {
            const int i = kp + SCAN_KP * m;
            if (i < d) S[(size_t)i * d + col] = sreg[m];
        }
}

// One warp per (token, head).
template <typename OT>
__global__ void __launch_bounds__(256)
wkv_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long ldg,
                  const float* __restrict__ norm_w, float eps, const int* __restrict__ seq_of_token, int num_tokens,
                  int heads, int d, OT* __restrict__ out) {
    pdl_sync();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)num_tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    const size_t base = (size_t)t * heads * d + (size_t)head * d;
    if (seq_of_token[t] < 0) {
        for (int e = lane; e < d; e += 32) st_f(out + base + e, 0.f);
        return;
    }
    float ss = 0.f;
    for (int e = lane; e < d; e += 32) {
        const float x = o[base + e];
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int e = lane; e < d; e += 32) {
        const float g = gate[(size_t)t * ldg + (size_t)head * d + e];
        st_f(out + base + e, o[base + e] * inv * norm_w[(size_t)head * d + e] * (g / (1.0f + expf(-g))));
    }
}

}  // namespace

// h: [T, width] 32-bit; mu: [streams, width]; state: per slot `width` floats at the start of a row of
// state_pitch floats; out: [streams, T, width] in out_dt; last32 (may be null): [T, width] 32-bit, receives
// the last blend instead of out.
MOE_API int moe_wkv_shift_mix(const float* h, const float* mu, int streams, float* state, long long state_pitch,
                              const int* seq_of_token, const int* pos, const int* cu_seqlens, const int* slots,
                              int num_tokens, int width, void* out, int out_dt, float* last32, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!h || !mu || !state || !out || streams <= 0 || width <= 0 || state_pitch < width) return (int)cudaErrorInvalidValue;
    if (out_dt == DT_F32)
        return launch_pdl(wkv_shift_mix_kernel<float>, dim3(num_tokens), 256, 0, stream, h, mu, streams, state,
                          state_pitch, seq_of_token, pos, cu_seqlens, slots, num_tokens, width, (float*)out, last32);
    return launch_pdl(wkv_shift_mix_kernel<__nv_bfloat16>, dim3(num_tokens), 256, 0, stream, h, mu, streams, state,
                      state_pitch, seq_of_token, pos, cu_seqlens, slots, num_tokens, width, (__nv_bfloat16*)out, last32);
}

// low: [T, rank] 32-bit; w2: [inner, rank]; w0: [inner]; out: [T, inner] 32-bit, the decay.
MOE_API int moe_wkv_decay(const float* low, const float* w2, const float* w0, int num_tokens, int inner, int rank,
                          float* out, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!low || !w2 || !w0 || !out || inner <= 0 || rank <= 0 || rank > MAX_RANK) return (int)cudaErrorInvalidValue;
    return launch_pdl(wkv_decay_kernel, dim3(num_tokens), 256, 0, stream, low, w2, w0, inner, rank, out);
}

// r, k, v, w (the decay): [T, heads * d] 32-bit with a row pitch of ld floats; u: [heads, d];
// state: per slot heads * d * d floats ([head][i][j]) at the start of a row of state_pitch floats;
// out: [T, heads * d] 32-bit (rows of no sequence are left alone).
MOE_API int moe_wkv_scan(const float* r, const float* k, const float* v, const float* w, long long ld,
                         const float* u, float* state, long long state_pitch, const int* cu_seqlens, const int* slots,
                         int num_seqs, int heads, int d, float* out, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (!r || !k || !v || !w || !u || !state || !out || heads <= 0 || d <= 0 || d > 256 ||
        ld < (long long)heads * d || state_pitch < (long long)heads * d * d || heads > 65535 || num_seqs > 65535)
        return (int)cudaErrorInvalidValue;
    const dim3 grid((d + SCAN_COLS - 1) / SCAN_COLS, heads, num_seqs);
    const size_t smem = (size_t)SCAN_TOK * 3 * d * sizeof(float);
#define SCAN(RPT_)                                                                                                \
    return launch_pdl(wkv_scan_kernel<RPT_>, grid, SCAN_THREADS, smem, stream, r, k, v, w, ld, u, state,            \
                      state_pitch, cu_seqlens, slots, heads, d, out)
    if (d <= 32) SCAN(4);
    if (d <= 64) SCAN(8);
    if (d <= 128) SCAN(16);
    SCAN(32);
#undef SCAN
}

// o: [T, heads * d] 32-bit; gate: the gate projection's output, 32-bit, row pitch ldg; norm_w: [heads * d];
// out: [T, heads * d] in out_dt.
MOE_API int moe_wkv_finish(const float* o, const float* gate, long long ldg, const float* norm_w, float eps,
                           const int* seq_of_token, int num_tokens, int heads, int d, void* out, int out_dt,
                           cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!o || !gate || !norm_w || !out || heads <= 0 || d <= 0 || ldg < (long long)heads * d)
        return (int)cudaErrorInvalidValue;
    const long long items = (long long)num_tokens * heads;
    const unsigned blocks = (unsigned)((items + 7) / 8);
    if (out_dt == DT_F32)
        return launch_pdl(wkv_finish_kernel<float>, dim3(blocks), 256, 0, stream, o, gate, ldg, norm_w, eps,
                          seq_of_token, num_tokens, heads, d, (float*)out);
    return launch_pdl(wkv_finish_kernel<__nv_bfloat16>, dim3(blocks), 256, 0, stream, o, gate, ldg, norm_w, eps,
                      seq_of_token, num_tokens, heads, d, (__nv_bfloat16*)out);
}
