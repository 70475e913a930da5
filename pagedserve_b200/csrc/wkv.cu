// Kernels of the linear-recurrence mixer with per-channel, data-dependent decay ("wkv").
//
// Per request the mixer keeps, in the request's slot, float32 state of fixed size:
//   S     [heads, d, d]   per head a matrix, key channel x value channel
//   last  [W]             the mixer's input at the request's newest token
// laid out as one row of `state` per slot: S first, `last` at prev_offset.
//
// token_shift_mix:  m_s[t] = x[t] + (x[t-1] - x[t]) * mu_s  for each of n_mix mixing vectors mu_s, where x[t-1] is
//                   `last` of the request's slot for the first token of an entry (zeros for a new request).
//                   Only reads the state; wkv_recurrence, which runs later in the step, stores the new `last`.
// wkv_recurrence:   per (entry, head), tokens in order:
//                     w_t = exp(-exp(decay_t))                               (float32)
//                     y_t[j] = sum_i r_t[i] * (S[i][j] + u[i] k_t[i] v_t[j])
//                     S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
//                   then y_t / sqrt(mean_j y_t[j]^2 + eps) * gain[j] * gate_t[j], rounded to the output type.
//                   Thread j of a CTA owns column j of S in registers; a token's r, k, w are staged in shared
//                   memory. Sums run over i in order: a token's result does not depend on what else is in the step.
//                   r, k, v, decay and gate are float32 whatever the compute type is.
#include "common.cuh"

namespace ps {

template <typename T>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ mu, int n_mix,
                       const float* __restrict__ state, long long state_stride, int prev_offset,
                       const int* __restrict__ token_item, const int* __restrict__ q_start,
                       const int* __restrict__ item_slot, T* __restrict__ out, long long mix_stride, int out_stride,
                       int W) {
    pdl_prologue();
    x = pdl_fresh(x);
    state = pdl_fresh(state);
    const int t = blockIdx.x;
    const int item = token_item[t];
    const bool first = (t == q_start[item]);
    const float* before = state + (long long)item_slot[item] * state_stride + prev_offset;
    const T* row = x + (size_t)t * x_stride;
    const T* row_before = x + (size_t)(t > 0 ? t - 1 : 0) * x_stride;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float now = to_float(row[c]);
        const float prev = first ? before[c] : to_float(row_before[c]);
        const float delta = prev - now;
        for (int s = 0; s < n_mix; ++s)
            out[(long long)s * mix_stride + (size_t)t * out_stride + c] = from_float<T>(fmaf(delta, mu[(size_t)s * W + c], now));
    }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(DMAX)
wkv_recurrence_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                      const float* __restrict__ decay, const float* __restrict__ gate, int ld,
                      const float* __restrict__ u, const float* __restrict__ gain, float eps,
                      const T* __restrict__ x, int x_stride, int W, float* __restrict__ state, long long state_stride,
                      int prev_offset, const int* __restrict__ q_start, const int* __restrict__ item_slot,
                      T* __restrict__ out, int out_stride, int heads, int d) {
    __shared__ float s_r[2][DMAX], s_k[2][DMAX], s_w[2][DMAX], s_u[DMAX];
    __shared__ float red[2][DMAX / 32];
    pdl_prologue();
    r = pdl_fresh(r); k = pdl_fresh(k); v = pdl_fresh(v); decay = pdl_fresh(decay); gate = pdl_fresh(gate);
    x = pdl_fresh(x);
    const int item = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
    const int begin = q_start[item], end = q_start[item + 1];
    if (begin >= end) return;
    const bool live = j < d;
    const int lane = j & 31, warp = j >> 5, warps = (d + 31) >> 5;
    float* row_state = state + (long long)item_slot[item] * state_stride;
    float* S = row_state + (long long)h * d * d;
    float col[DMAX];
#pragma unroll
    for (int i = 0; i < DMAX; ++i) col[i] = (live && i < d) ? S[(size_t)i * d + j] : 0.f;
    const int c = h * d + j;
    s_u[j] = live ? u[c] : 0.f;
    const float gain_j = live ? gain[c] : 0.f;
    const float inv_d = 1.0f / (float)d;
    for (int t = begin; t < end; ++t) {
        const int b = (t - begin) & 1;
        const size_t at = (size_t)t * ld + c;
        float vj = 0.f;
        if (live) {
            s_r[b][j] = r[at];
            s_k[b][j] = k[at];
            s_w[b][j] = expf(-expf(decay[at]));
            vj = v[at];
        }
        __syncthreads();                      // the token's r, k, w are staged (the other buffer is the token before)
        float y = 0.f;
#pragma unroll
        for (int i = 0; i < DMAX; ++i) {
            if (i < d) {
                const float kv = s_k[b][i] * vj;
                y = fmaf(s_r[b][i], fmaf(s_u[i], kv, col[i]), y);
                col[i] = fmaf(s_w[b][i], col[i], kv);
            }
        }
        const float sq = warp_sum(live ? y * y : 0.f);
        if (lane == 0) red[b][warp] = sq;
        __syncthreads();
        float total = 0.f;
        for (int w = 0; w < warps; ++w) total += red[b][w];
        if (live)
            out[(size_t)t * out_stride + c] = from_float<T>(y * rsqrtf(total * inv_d + eps) * gain_j * gate[at]);
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DMAX; ++i)
            if (i < d) S[(size_t)i * d + j] = col[i];
    }
    // the entry's newest input becomes `last` (each head's CTA copies a share of the row)
    const T* newest = x + (size_t)(end - 1) * x_stride;
    float* last = row_state + prev_offset;
    for (int w = h * DMAX + j; w < W; w += heads * DMAX) last[w] = to_float(newest[w]);
}

template <typename T, int DMAX>
int launch_wkv(const float* r, const float* k, const float* v, const float* decay, const float* gate, int ld,
               const float* u, const float* gain, float eps, const void* x, int x_stride, int W, float* state,
               long long state_stride, int prev_offset, const int* q_start, const int* item_slot, void* out,
               int out_stride, int n_items, int heads, int d, cudaStream_t s) {
    return launch_pdl(wkv_recurrence_kernel<T, DMAX>, dim3(n_items, heads), dim3(DMAX), 0, s, r, k, v, decay, gate, ld, u,
                      gain, eps, (const T*)x, x_stride, W, state, state_stride, prev_offset, q_start, item_slot,
                      (T*)out, out_stride, heads, d);
}

template <typename T>
int pick_wkv(const float* r, const float* k, const float* v, const float* decay, const float* gate, int ld,
             const float* u, const float* gain, float eps, const void* x, int x_stride, int W, float* state,
             long long state_stride, int prev_offset, const int* q_start, const int* item_slot, void* out,
             int out_stride, int n_items, int heads, int d, cudaStream_t s) {
#define PS_WKV(DM)                                                                                                  \
    return launch_wkv<T, DM>(r, k, v, decay, gate, ld, u, gain, eps, x, x_stride, W, state, state_stride, prev_offset, \
                             q_start, item_slot, out, out_stride, n_items, heads, d, s)
    if (d <= 32) PS_WKV(32);
    if (d <= 64) PS_WKV(64);
    if (d <= 96) PS_WKV(96);
    PS_WKV(128);
#undef PS_WKV
}

}  // namespace ps

// out[s][t] = x[t] + (x[t-1] - x[t]) * mu[s]; out is [n_mix] blocks of mix_stride elements, rows of out_stride.
PS_EXPORT int ps_token_shift_mix(const void* x, int x_stride, const float* mu, int n_mix, const float* state,
                                 long long state_stride, int prev_offset, const int* token_item, const int* q_start,
                                 const int* item_slot, void* out, long long mix_stride, int out_stride, int T, int W,
                                 int dtype, void* stream) {
    if (T <= 0) return PS_OK;
    if (!x || !mu || !state || !token_item || !q_start || !item_slot || !out || W <= 0 || n_mix <= 0)
        return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = W >= 256 ? 256 : 128;
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::token_shift_mix_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)x, x_stride,
                              mu, n_mix, state, state_stride, prev_offset, token_item, q_start, item_slot, (float*)out,
                              mix_stride, out_stride, W);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::token_shift_mix_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s,
                              (const __nv_bfloat16*)x, x_stride, mu, n_mix, state, state_stride, prev_offset,
                              token_item, q_start, item_slot, (__nv_bfloat16*)out, mix_stride, out_stride, W);
    return PS_ERR_UNSUPPORTED;
}

// r, k, v, decay, gate: float32 [T, heads * d] with row stride ld. x: the mixer's input [T, W] (dtype), whose newest
// row of each entry is stored as the slot's `last`. out: [T, heads * d] (dtype).
PS_EXPORT int ps_wkv_recurrence(const float* r, const float* k, const float* v, const float* decay, const float* gate,
                                int ld, const float* u, const float* gain, float eps, const void* x, int x_stride,
                                int W, float* state, long long state_stride, int prev_offset, const int* q_start,
                                const int* item_slot, void* out, int out_stride, int n_items, int heads, int d,
                                int dtype, void* stream) {
    if (n_items <= 0) return PS_OK;
    if (!r || !k || !v || !decay || !gate || !u || !gain || !x || !state || !q_start || !item_slot || !out)
        return PS_ERR_BAD_ARGUMENT;
    if (heads <= 0 || heads > 65535 || d <= 0 || W <= 0) return PS_ERR_BAD_ARGUMENT;
    if (d > 128) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PS_F32)
        return ps::pick_wkv<float>(r, k, v, decay, gate, ld, u, gain, eps, x, x_stride, W, state, state_stride,
                                   prev_offset, q_start, item_slot, out, out_stride, n_items, heads, d, s);
    if (dtype == PS_BF16)
        return ps::pick_wkv<__nv_bfloat16>(r, k, v, decay, gate, ld, u, gain, eps, x, x_stride, W, state, state_stride,
                                           prev_offset, q_start, item_slot, out, out_stride, n_items, heads, d, s);
    return PS_ERR_UNSUPPORTED;
}
