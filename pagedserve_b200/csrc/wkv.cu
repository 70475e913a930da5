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
//                            = sum_i r_t[i] S[i][j]  +  v_t[j] * sum_i r_t[i] u[i] k_t[i]
//                     S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
//                   then y_t / sqrt(mean_j y_t[j]^2 + eps) * gain[j] * gate_t[j], rounded to the output type.
//                   One CTA per (entry, head); S lives in registers, a block of rows x 4 columns per thread;
//                   tokens are brought into shared memory in chunks, one chunk ahead of the one being computed. Sums run in a fixed order: a token's result does not depend on what else is in the
//                   step, nor on where a prompt was cut.
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
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        const float now = to_float(row[c]);
        const float prev = first ? before[c] : to_float(row_before[c]);
        const float delta = prev - now;
        for (int s = 0; s < n_mix; ++s)
            out[(long long)s * mix_stride + (size_t)t * out_stride + c] = from_float<T>(fmaf(delta, mu[(size_t)s * W + c], now));
    }
}

// the sum over each half of a warp (lanes 0..15, lanes 16..31), in a fixed order
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ void wkv_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void wkv_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}

// Shared memory of one CTA, in floats: two buffers of CH tokens (r, k, w in rows of PARTS runs; v, gate in plain
// rows), the chunk's unnormalised outputs, its bonus numbers, and the head's u and gain.
template <int DMAX>
struct WkvLayout {
    static constexpr int COLS = 4;                                      // columns of S per thread
    static constexpr int IQ = DMAX > 64 ? 8 : 4;                        // rows of S per thread
    static constexpr int PARTS = DMAX / IQ;                             // threads that share a column: 8 or 16
    static constexpr int RUN = IQ == 4 ? 4 : IQ + 4;                    // a part's run of a row, padded against bank conflicts
    static constexpr int ROW = PARTS * RUN;
    static constexpr int CH = DMAX > 64 ? 8 : 16;                       // tokens per chunk
    static constexpr int THREADS = (DMAX / COLS) * PARTS, WARPS = THREADS / 32;
    static constexpr int BUF = 3 * CH * ROW + 2 * CH * DMAX;
    static constexpr int Y = 2 * BUF, BONUS = Y + CH * DMAX, U = BONUS + CH, GAIN = U + DMAX, FLOATS = GAIN + DMAX;
    static constexpr size_t BYTES = (size_t)FLOATS * 4;
    static_assert(PARTS == 8 || PARTS == 16, "the sum over parts is a butterfly inside a warp");
};

template <typename T, int DMAX>
__global__ void __launch_bounds__(WkvLayout<DMAX>::THREADS)
wkv_recurrence_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                      const float* __restrict__ decay, const float* __restrict__ gate, int ld,
                      const float* __restrict__ u, const float* __restrict__ gain, float eps,
                      const T* __restrict__ x, int x_stride, int W, float* __restrict__ state, long long state_stride,
                      int prev_offset, const int* __restrict__ q_start, const int* __restrict__ item_slot,
                      T* __restrict__ out, int out_stride, int heads, int d) {
    // Thread (group, part) holds a block of S in registers: rows part * IQ .. + IQ - 1 of the four columns
    // 4 * group .. + 3, so that a token's r, k, w, read from shared memory, are used four times each. The PARTS
    // threads of a group are neighbours in a warp and add their partial sums up with shuffles. Tokens come in
    // chunks of CH through two buffers (asynchronous copies, one chunk ahead); inside a chunk the warps run
    // without barriers: the head norm, which needs all columns of a token, runs once per chunk over the outputs
    // kept in shared memory.
    using L = WkvLayout<DMAX>;
    constexpr int IQ = L::IQ, PARTS = L::PARTS, RUN = L::RUN, ROW = L::ROW, CH = L::CH, THREADS = L::THREADS,
                  WARPS = L::WARPS, Q4 = IQ / 4;
    extern __shared__ __align__(16) float wkv_smem[];
    float* const s_y = wkv_smem + L::Y;
    float* const s_bonus = wkv_smem + L::BONUS;
    float* const s_u = wkv_smem + L::U;
    float* const s_gain = wkv_smem + L::GAIN;
    const int item = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int begin = q_start[item], end = q_start[item + 1];
    if (begin >= end) return;
    const int part = tid % PARTS, j0 = (tid / PARTS) * 4, i0 = part * IQ;
    const int lane = tid & 31, warp = tid >> 5;
    // channels past d stay zero in both buffers: they add nothing to any sum and keep their (zero) entries of S
    if (d < DMAX)
        for (int e = tid; e < 2 * L::BUF; e += THREADS) wkv_smem[e] = 0.f;
    for (int i = tid; i < DMAX; i += THREADS) {
        s_u[i] = i < d ? u[h * d + i] : 0.f;
        s_gain[i] = i < d ? gain[h * d + i] : 0.f;
    }
    __syncthreads();
    pdl_prologue();
    r = pdl_fresh(r); k = pdl_fresh(k); v = pdl_fresh(v); decay = pdl_fresh(decay); gate = pdl_fresh(gate);
    x = pdl_fresh(x);
    const bool wide = (d & 3) == 0 && (ld & 3) == 0 &&
                      ((((uintptr_t)r | (uintptr_t)k | (uintptr_t)v | (uintptr_t)decay | (uintptr_t)gate) & 15) == 0);
    const int n_chunks = (end - begin + CH - 1) / CH;
    auto issue = [&](int chunk) {
        float* buf = wkv_smem + (chunk & 1) * L::BUF;
        const int t0 = begin + chunk * CH, n = min(CH, end - t0);
        if (wide) {
            // 16-byte pieces: a thread's place in a row is fixed, its token moves by THREADS / (DMAX / 4)
            constexpr int PIECES = DMAX / 4;
            const int i = (tid % PIECES) << 2;
            for (int tt = tid / PIECES; tt < n && i < d; tt += THREADS / PIECES) {
                const size_t at = (size_t)(t0 + tt) * ld + h * d + i;
                const int padded = tt * ROW + (i / IQ) * RUN + (i % IQ);
                wkv_copy16(buf + padded, r + at);
                wkv_copy16(buf + CH * ROW + padded, k + at);
                wkv_copy16(buf + 2 * CH * ROW + padded, decay + at);
                wkv_copy16(buf + 3 * CH * ROW + tt * DMAX + i, v + at);
                wkv_copy16(buf + 3 * CH * ROW + CH * DMAX + tt * DMAX + i, gate + at);
            }
        } else {
            for (int e = tid; e < n * d; e += THREADS) {
                const int tt = e / d, i = e - tt * d;
                const size_t at = (size_t)(t0 + tt) * ld + h * d + i;
                const int padded = tt * ROW + (i / IQ) * RUN + (i % IQ);
                wkv_copy4(buf + padded, r + at);
                wkv_copy4(buf + CH * ROW + padded, k + at);
                wkv_copy4(buf + 2 * CH * ROW + padded, decay + at);
                wkv_copy4(buf + 3 * CH * ROW + tt * DMAX + i, v + at);
                wkv_copy4(buf + 3 * CH * ROW + CH * DMAX + tt * DMAX + i, gate + at);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0);
    float* row_state = state + (long long)item_slot[item] * state_stride;
    float* S = row_state + (long long)h * d * d;
    const bool wide_state = (d & 3) == 0 && (((uintptr_t)S) & 15) == 0;
    float s[IQ][4];                                           // s[ii][c] = S[i0 + ii][j0 + c]
#pragma unroll
    for (int ii = 0; ii < IQ; ++ii) {
        const int i = i0 + ii;
        if (wide_state && i < d && j0 < d) {
            const float4 got = *reinterpret_cast<const float4*>(S + (size_t)i * d + j0);
            s[ii][0] = got.x; s[ii][1] = got.y; s[ii][2] = got.z; s[ii][3] = got.w;
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) s[ii][c] = (i < d && j0 + c < d) ? S[(size_t)i * d + j0 + c] : 0.f;
        }
    }
    // after the butterfly below, a thread holds the sum of column j0 + mine
    const int mine = 2 * (part & 1) + ((part >> 1) & 1);
    const float inv_d = 1.0f / (float)d;
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        float* buf = wkv_smem + (chunk & 1) * L::BUF;
        float* s_r = buf;
        float* s_k = buf + CH * ROW;
        float* s_w = buf + 2 * CH * ROW;
        const float* s_v = buf + 3 * CH * ROW;
        const float* s_g = s_v + CH * DMAX;
        const int t0 = begin + chunk * CH, n = min(CH, end - t0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                      // everybody's copies of this chunk have landed, and
        if (chunk + 1 < n_chunks) issue(chunk + 1);           // nobody reads the other buffer any more
        // decay arguments become decays, in place; one number per token for the bonus:
        // y_j gets v_j * sum_i r_i u_i k_i, the part of the sum that the token's own k v^T contributes
        {
            // a thread's channel is fixed (compile-time place in the padded row), its token moves by THREADS / DMAX
            constexpr int ROUNDS = (CH * DMAX + THREADS - 1) / THREADS;
            const int i = tid % DMAX, padded_i = (i / IQ) * RUN + (i % IQ);
            float arg[ROUNDS];
#pragma unroll
            for (int k = 0; k < ROUNDS; ++k) {
                const int tt = tid / DMAX + k * (THREADS / DMAX);
                arg[k] = (tt < n && i < d) ? s_w[tt * ROW + padded_i] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < ROUNDS; ++k) arg[k] = expf(-expf(arg[k]));
#pragma unroll
            for (int k = 0; k < ROUNDS; ++k) {
                const int tt = tid / DMAX + k * (THREADS / DMAX);
                if (tt < n && i < d) s_w[tt * ROW + padded_i] = arg[k];
            }
        }
        // (sixteen lanes per token, so that a warp works on two tokens at a time)
        for (int first = 2 * warp; first < n; first += 2 * WARPS) {
            const int tt = first + (lane >> 4);
            float p = 0.f;
            if (tt < n) {
                float rk[DMAX / 16];
#pragma unroll
                for (int k = 0; k < DMAX / 16; ++k) {
                    const int i = (lane & 15) + 16 * k;
                    const int padded = tt * ROW + (i / IQ) * RUN + (i % IQ);
                    rk[k] = i < d ? s_r[padded] * s_u[i] * s_k[padded] : 0.f;
                }
#pragma unroll
                for (int k = 0; k < DMAX / 16; ++k) p += rk[k];
            }
            p = half_warp_sum(p);
            if ((lane & 15) == 0 && tt < n) s_bonus[tt] = p;
        }
        __syncthreads();
        // The chunk's tokens in order. Nothing but registers is written here, so that the reads of the tokens
        // ahead can be scheduled early; each token leaves this thread's share of its four outputs in y[tt].
        float y[CH][4];
        auto token = [&](int tt) {
            const float4 vv = *reinterpret_cast<const float4*>(s_v + tt * DMAX + j0);
            const float vc[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int q = 0; q < Q4; ++q) {
                const float4 rr = *reinterpret_cast<const float4*>(s_r + tt * ROW + part * RUN + 4 * q);
                const float4 kk = *reinterpret_cast<const float4*>(s_k + tt * ROW + part * RUN + 4 * q);
                const float4 ww = *reinterpret_cast<const float4*>(s_w + tt * ROW + part * RUN + 4 * q);
                const float ri[4] = {rr.x, rr.y, rr.z, rr.w}, ki[4] = {kk.x, kk.y, kk.z, kk.w},
                            wi[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        y[tt][c] = fmaf(ri[e], s[4 * q + e][c], y[tt][c]);
                        s[4 * q + e][c] = fmaf(wi[e], s[4 * q + e][c], ki[e] * vc[c]);
                    }
                }
            }
        };
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) y[tt][0] = y[tt][1] = y[tt][2] = y[tt][3] = 0.f;
        if (n == CH) {
            // a full chunk is straight-line code: reads of later tokens move ahead of the arithmetic of earlier ones
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) token(tt);
        } else {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt)
                if (tt < n) token(tt);
        }
        // The sums over the parts, in a fixed order, for all tokens of the chunk at once: at every step a thread
        // passes half of what it holds to a neighbour and adds up the other half. Bits 0 and 1 of the part choose
        // the column, bits 2 and 3 the tokens that stay with a thread.
        const bool bit0 = part & 1, bit1 = (part >> 1) & 1, bit2 = (part >> 2) & 1, bit3 = (part >> 3) & 1;
        float a[CH][2];
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float keep = bit0 ? y[tt][2 + c] : y[tt][c], send = bit0 ? y[tt][c] : y[tt][2 + c];
                a[tt][c] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
            }
        }
        float b[CH];
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
            const float keep = bit1 ? a[tt][1] : a[tt][0], send = bit1 ? a[tt][0] : a[tt][1];
            b[tt] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        float c2[CH / 2];
#pragma unroll
        for (int q = 0; q < CH / 2; ++q) {
            const float keep = bit2 ? b[q + CH / 2] : b[q], send = bit2 ? b[q] : b[q + CH / 2];
            c2[q] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        }
        const int col = j0 + mine;
        if constexpr (PARTS == 16) {
#pragma unroll
            for (int q = 0; q < CH / 4; ++q) {
                const float keep = bit3 ? c2[q + CH / 4] : c2[q], send = bit3 ? c2[q] : c2[q + CH / 4];
                const float total = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                const int tt = bit2 * (CH / 2) + bit3 * (CH / 4) + q;
                if (tt < n) s_y[tt * DMAX + col] = fmaf(s_v[tt * DMAX + col], s_bonus[tt], total);
            }
        } else {
#pragma unroll
            for (int q = 0; q < CH / 2; ++q) {
                const int tt = bit2 * (CH / 2) + q;
                if (tt < n) s_y[tt * DMAX + col] = fmaf(s_v[tt * DMAX + col], s_bonus[tt], c2[q]);
            }
        }
        __syncthreads();
        // the head norm, the gain and the gate for the chunk's tokens: sixteen lanes per token
        for (int first = 2 * warp; first < n; first += 2 * WARPS) {
            const int tt = first + (lane >> 4);
            const bool valid = tt < n;
            float mine_y[DMAX / 16], factor[DMAX / 16], sq = 0.f;
#pragma unroll
            for (int k = 0; k < DMAX / 16; ++k) {
                const int i = (lane & 15) + 16 * k;
                const bool in = valid && i < d;
                mine_y[k] = in ? s_y[tt * DMAX + i] : 0.f;
                factor[k] = in ? s_gain[i] * s_g[tt * DMAX + i] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < DMAX / 16; ++k) sq = fmaf(mine_y[k], mine_y[k], sq);
            const float scale = rsqrtf(half_warp_sum(sq) * inv_d + eps);
            if (valid) {
                T* row = out + (size_t)(t0 + tt) * out_stride + h * d;
#pragma unroll
                for (int k = 0; k < DMAX / 16; ++k) {
                    const int i = (lane & 15) + 16 * k;
                    if (i < d) row[i] = from_float<T>(mine_y[k] * scale * factor[k]);
                }
            }
        }
    }
#pragma unroll
    for (int ii = 0; ii < IQ; ++ii) {
        const int i = i0 + ii;
        if (wide_state && i < d && j0 < d) {
            *reinterpret_cast<float4*>(S + (size_t)i * d + j0) = make_float4(s[ii][0], s[ii][1], s[ii][2], s[ii][3]);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (i < d && j0 + c < d) S[(size_t)i * d + j0 + c] = s[ii][c];
        }
    }
    // the entry's newest input becomes `last` (each head's CTA copies a share of the row)
    const T* newest = x + (size_t)(end - 1) * x_stride;
    float* last = row_state + prev_offset;
    for (int w = h * THREADS + tid; w < W; w += heads * THREADS) last[w] = to_float(newest[w]);
}

template <typename T, int DMAX>
int launch_wkv(const float* r, const float* k, const float* v, const float* decay, const float* gate, int ld,
               const float* u, const float* gain, float eps, const void* x, int x_stride, int W, float* state,
               long long state_stride, int prev_offset, const int* q_start, const int* item_slot, void* out,
               int out_stride, int n_items, int heads, int d, cudaStream_t s) {
    using L = WkvLayout<DMAX>;
    auto kernel = wkv_recurrence_kernel<T, DMAX>;
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, L::BYTES, raised)) return PS_ERR_LAUNCH;
    return launch_pdl(kernel, dim3(n_items, heads), dim3(L::THREADS), L::BYTES, s, r, k, v, decay, gate, ld,
                      u, gain, eps, (const T*)x, x_stride, W, state, state_stride, prev_offset, q_start, item_slot,
                      (T*)out, out_stride, heads, d);
}

// eight consecutive elements as floats (16-byte loads; the address is 16-byte aligned)
__device__ __forceinline__ void load8(const float* p, float (&o)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&o)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* pair = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(pair[i]);
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}

// wkv_prepare: everything between the residual stream and the mixer's large products, for one token per CTA:
//   x[t]   = rms_norm(h[t]) * gain, rounded to the compute type (as the norm kernel rounds it)
//   m_s[t] = x[t] + (x[t-1] - x[t]) * mu_s for s = 0 .. 3, written as blends; x[t] itself is written too
//   m_w    = the fifth blend, kept in shared memory
//   low    = tanh(W1 m_w)                      (rank numbers, rounded to the compute type)
//   decay[t] = W2 low + w0                     (float32; the argument of exp(-exp(.)))
// x[t-1] of an entry's first token is the slot's `last`; other tokens norm the row before their own themselves.
template <typename T>
__global__ void __launch_bounds__(256)
wkv_prepare_kernel(const float* __restrict__ h, int ld_h, const float* __restrict__ gain, float eps,
                   const float* __restrict__ mu, const float* __restrict__ state, long long state_stride,
                   int prev_offset, const int* __restrict__ token_item, const int* __restrict__ q_start,
                   const int* __restrict__ item_slot, const T* __restrict__ w1, int ld_w1, int rank,
                   const T* __restrict__ w2, int ld_w2, const float* __restrict__ w0, int inner,
                   T* __restrict__ blends, long long mix_stride, int ld_blend, float* __restrict__ decay,
                   int ld_decay, int W) {
    extern __shared__ __align__(16) float prep_smem[];
    float* const m_w = prep_smem;                       // [W]
    float* const low = prep_smem + W;                   // [rank]
    __shared__ float red[2][8];
    pdl_prologue();
    h = pdl_fresh(h);
    state = pdl_fresh(state);
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int item = token_item[t];
    const bool first = (t == q_start[item]);
    const float* before = state + (long long)item_slot[item] * state_stride + prev_offset;
    const float* row = h + (size_t)t * ld_h;
    const float* row_before = h + (size_t)(t > 0 ? t - 1 : 0) * ld_h;
    float ss = 0.f, ss_before = 0.f;
    for (int c = tid; c < W; c += 256) {
        const float a = row[c];
        ss = fmaf(a, a, ss);
        if (!first) {
            const float b = row_before[c];
            ss_before = fmaf(b, b, ss_before);
        }
    }
    ss = warp_sum(ss);
    ss_before = warp_sum(ss_before);
    if (lane == 0) { red[0][warp] = ss; red[1][warp] = ss_before; }
    __syncthreads();
    float total = 0.f, total_before = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { total += red[0][w]; total_before += red[1][w]; }
    const float scale = rsqrtf(total / (float)W + eps), scale_before = rsqrtf(total_before / (float)W + eps);
    // every CTA of a token (gridDim.y of them when the step has few tokens) makes the whole fifth blend, but
    // writes only its share of the other blends and of the decay's argument
    for (int c = tid; c < W; c += 256) {
        const T now_t = from_float<T>(row[c] * scale * gain[c]);
        const float now = to_float(now_t);
        const float prev = first ? before[c] : to_float(from_float<T>(row_before[c] * scale_before * gain[c]));
        const float delta = prev - now;
        if ((c >> 8) % gridDim.y == blockIdx.y) {
#pragma unroll
            for (int s = 0; s < 4; ++s)
                blends[(long long)s * mix_stride + (size_t)t * ld_blend + c] = from_float<T>(fmaf(delta, mu[(size_t)s * W + c], now));
            blends[4 * mix_stride + (size_t)t * ld_blend + c] = now_t;
        }
        m_w[c] = to_float(from_float<T>(fmaf(delta, mu[(size_t)4 * W + c], now)));
    }
    __syncthreads();
    const bool wide1 = (W & 7) == 0 && (ld_w1 & 7) == 0 && (((uintptr_t)w1) & 15) == 0;
    for (int rho = warp; rho < rank; rho += 8) {
        const T* wr = w1 + (size_t)rho * ld_w1;
        float acc = 0.f;
        if (wide1) {
            for (int c = lane * 8; c < W; c += 256) {
                float w8[8];
                load8(wr + c, w8);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc = fmaf(w8[i], m_w[c + i], acc);
            }
        } else {
            for (int c = lane; c < W; c += 32) acc = fmaf(to_float(wr[c]), m_w[c], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) low[rho] = to_float(from_float<T>(tanhf(acc)));
    }
    __syncthreads();
    const bool wide2 = (rank & 7) == 0 && (ld_w2 & 7) == 0 && (((uintptr_t)w2) & 15) == 0;
    for (int c = blockIdx.y * 256 + tid; c < inner; c += gridDim.y * 256) {
        const T* wr = w2 + (size_t)c * ld_w2;
        float acc = 0.f;
        if (wide2) {
            for (int rho = 0; rho < rank; rho += 8) {
                float w8[8];
                load8(wr + rho, w8);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc = fmaf(w8[i], low[rho + i], acc);
            }
        } else {
            for (int rho = 0; rho < rank; ++rho) acc = fmaf(to_float(wr[rho]), low[rho], acc);
        }
        decay[(size_t)t * ld_decay + c] = acc + w0[c];
    }
}

template <typename T>
int launch_wkv_prepare(const float* h, int ld_h, const float* gain, float eps, const float* mu, const float* state,
                       long long state_stride, int prev_offset, const int* token_item, const int* q_start,
                       const int* item_slot, const void* w1, int ld_w1, int rank, const void* w2, int ld_w2,
                       const float* w0, int inner, void* blends, long long mix_stride, int ld_blend, float* decay,
                       int ld_decay, int n_tokens, int W, cudaStream_t s) {
    auto kernel = wkv_prepare_kernel<T>;
    const size_t smem = (size_t)(W + rank) * sizeof(float);
    static size_t raised[MAX_DEVICES] = {0};
    if (!ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;
    // a step of few tokens is bound by the chain of one CTA's phases: share a token's writes out over several
    const int widest = W > inner ? W : inner;
    const int split = n_tokens >= 512 ? 1 : (widest + 255) / 256;
    return launch_pdl(kernel, dim3(n_tokens, split), dim3(256), smem, s, h, ld_h, gain, eps, mu, state, state_stride,
                      prev_offset, token_item, q_start, item_slot, (const T*)w1, ld_w1, rank, (const T*)w2, ld_w2, w0,
                      inner, (T*)blends, mix_stride, ld_blend, decay, ld_decay, W);
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
    // few tokens (decode): a row is shared out over several CTAs, one column per thread
    const int split = T >= 512 ? 1 : (W + threads - 1) / threads;
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::token_shift_mix_kernel<float>, dim3(T, split), dim3(threads), 0, s, (const float*)x, x_stride,
                              mu, n_mix, state, state_stride, prev_offset, token_item, q_start, item_slot, (float*)out,
                              mix_stride, out_stride, W);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::token_shift_mix_kernel<__nv_bfloat16>, dim3(T, split), dim3(threads), 0, s,
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

// The norm of the residual rows, the five blends (four written to `blends` [5][T, W] together with the normed
// rows themselves in block 4; the fifth used in place), and the decay's argument W2 tanh(W1 m_w) + w0 (float32).
// h: float32 [T, W]; gain: the RMS norm's gain; w1 [rank, W], w2 [inner, rank] in the compute type.
PS_EXPORT int ps_wkv_prepare(const float* h, int ld_h, const float* gain, float eps, const float* mu,
                             const float* state, long long state_stride, int prev_offset, const int* token_item,
                             const int* q_start, const int* item_slot, const void* w1, int ld_w1, int rank,
                             const void* w2, int ld_w2, const float* w0, int inner, void* blends,
                             long long mix_stride, int ld_blend, float* decay, int ld_decay, int T, int W, int dtype,
                             void* stream) {
    if (T <= 0) return PS_OK;
    if (!h || !gain || !mu || !state || !token_item || !q_start || !item_slot || !w1 || !w2 || !w0 || !blends || !decay)
        return PS_ERR_BAD_ARGUMENT;
    if (W <= 0 || rank <= 0 || inner <= 0) return PS_ERR_BAD_ARGUMENT;
    if ((size_t)(W + rank) * sizeof(float) > 200 * 1024) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PS_F32)
        return ps::launch_wkv_prepare<float>(h, ld_h, gain, eps, mu, state, state_stride, prev_offset, token_item,
                                             q_start, item_slot, w1, ld_w1, rank, w2, ld_w2, w0, inner, blends,
                                             mix_stride, ld_blend, decay, ld_decay, T, W, s);
    if (dtype == PS_BF16)
        return ps::launch_wkv_prepare<__nv_bfloat16>(h, ld_h, gain, eps, mu, state, state_stride, prev_offset,
                                                     token_item, q_start, item_slot, w1, ld_w1, rank, w2, ld_w2, w0,
                                                     inner, blends, mix_stride, ld_blend, decay, ld_decay, T, W, s);
    return PS_ERR_UNSUPPORTED;
}
