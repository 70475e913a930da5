// Routed experts: the router and the gated inner activation.
//
// moe_route, one warp per token, float32 throughout:
//     z = W_router h                    (E numbers; the operands may be bfloat16, sums are float32)
//     s = softmax(z) over all E experts
//     with groups: the experts are `groups` runs of E / groups neighbours; a group's mark is its largest s; only
//     experts of the `keep` groups with the largest marks stand for election
//     the `top` largest s among them are chosen (ties: the lower index), and their weights are s / (sum of the
//     chosen s + 1e-20)
//     shared gate: sigmoid(w_sg . h), one number per token (where the layer has a shared expert)
// Results: dense weights [T, E] (0 where an expert is not chosen), the chosen experts and their weights
// [T, top], and the shared gate [T].
//
// moe_gate_mul: inner[t, c] = silu(gate[t, c]) * up[t, c] * weight[t, expert of column c], where gate and up are
// the two halves of one stacked product over all experts' columns, columns [e * F, (e + 1) * F) belong to expert
// e and the columns from E * F on to the shared expert (weight = the shared gate).  Products in float32, rounded
// once.
#include "common.cuh"

namespace ps {

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_route_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ router, int router_stride,
                 const T* __restrict__ shared_gate_w, float* __restrict__ dense, int* __restrict__ chosen,
                 float* __restrict__ chosen_w, float* __restrict__ shared_gate, int tokens, int W, int E, int top,
                 int groups, int keep) {
    pdl_prologue();
    x = pdl_fresh(x);
    __shared__ float score[MOE_WARPS][MOE_MAX_EXPERTS];
    __shared__ unsigned char open[MOE_WARPS][MOE_MAX_EXPERTS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * MOE_WARPS + warp;
    if (t >= tokens) return;
    const T* row = x + (size_t)t * x_stride;
    for (int e = 0; e < E; ++e) {
        const T* w = router + (size_t)e * router_stride;
        float acc = 0.f;
        for (int j = lane; j < W; j += 32) acc = fmaf(to_float(row[j]), to_float(w[j]), acc);
        acc = warp_sum(acc);
        if (lane == 0) score[warp][e] = acc;
    }
    if (shared_gate_w) {
        float acc = 0.f;
        for (int j = lane; j < W; j += 32) acc = fmaf(to_float(row[j]), to_float(shared_gate_w[j]), acc);
        acc = warp_sum(acc);
        if (lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-acc));
    }
    __syncwarp();
    // softmax over all experts
    float top_z = -INFINITY;
    for (int e = lane; e < E; e += 32) top_z = fmaxf(top_z, score[warp][e]);
    top_z = warp_max(top_z);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(score[warp][e] - top_z);
        score[warp][e] = v;
        sum += v;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        score[warp][e] *= inv;
        open[warp][e] = 1;
        dense[(size_t)t * E + e] = 0.f;
    }
    __syncwarp();
    if (lane == 0) {
        float* s = score[warp];
        unsigned char* ok = open[warp];
        if (groups > 1 && keep < groups) {
            // close every group but the `keep` best: repeatedly drop the group with the lowest mark
            // (ties: the higher index goes first, so that the lower index wins as in the election below)
            const int per = E / groups;
            for (int drop = 0; drop < groups - keep; ++drop) {
                int worst = -1;
                float worst_mark = INFINITY;
                for (int g = 0; g < groups; ++g) {
                    if (!ok[g * per]) continue;
                    float mark = -INFINITY;
                    for (int j = 0; j < per; ++j) mark = fmaxf(mark, s[g * per + j]);
                    if (mark <= worst_mark) {
                        worst_mark = mark;
                        worst = g;
                    }
                }
                if (worst < 0) break;
                for (int j = 0; j < per; ++j) ok[worst * per + j] = 0;
            }
        }
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float best_s = -INFINITY;
            for (int e = 0; e < E; ++e)
                if (ok[e] && s[e] > best_s) {
                    best_s = s[e];
                    best = e;
                }
            if (best < 0) {                      // fewer open experts than `top`: the rest get no weight
                chosen[(size_t)t * top + k] = -1;
                chosen_w[(size_t)t * top + k] = 0.f;
                continue;
            }
            ok[best] = 0;
            chosen[(size_t)t * top + k] = best;
            chosen_w[(size_t)t * top + k] = best_s;
            total += best_s;
        }
        const float scale = 1.0f / (total + 1e-20f);
        for (int k = 0; k < top; ++k) {
            const int e = chosen[(size_t)t * top + k];
            if (e < 0) continue;
            const float w = chosen_w[(size_t)t * top + k] * scale;
            chosen_w[(size_t)t * top + k] = w;
            dense[(size_t)t * E + e] = w;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_mul_kernel(const T* __restrict__ gate_up, int gu_stride, const float* __restrict__ dense,
                    const float* __restrict__ shared_gate, T* __restrict__ inner, int inner_stride, int tokens,
                    int columns, int E, int F) {
    pdl_prologue();
    gate_up = pdl_fresh(gate_up);
    dense = pdl_fresh(dense);
    shared_gate = pdl_fresh(shared_gate);
    const long long total = (long long)tokens * columns;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / columns), c = (int)(i - (long long)t * columns);
        const int e = c / F;
        const float w = e < E ? dense[(size_t)t * E + e] : shared_gate[t];
        float v = 0.f;
        if (w != 0.f) {
            const T* row = gate_up + (size_t)t * gu_stride;
            v = silu(to_float(row[c])) * to_float(row[columns + c]) * w;
        }
        inner[(size_t)t * inner_stride + c] = from_float<T>(v);
    }
}

}  // namespace ps

// x [T, W] rows of the compute type; router [E, W]; shared_gate_w [W] or null; dense float32 [T, E];
// chosen int32 [T, top]; chosen_w float32 [T, top]; shared_gate float32 [T] (written only with shared_gate_w).
PS_EXPORT int ps_moe_route(const void* x, int x_stride, const void* router, int router_stride,
                           const void* shared_gate_w, float* dense, int* chosen, float* chosen_w, float* shared_gate,
                           int T, int W, int E, int top, int groups, int keep, int dtype, void* stream) {
    if (T <= 0) return PS_OK;
    if (W <= 0 || E <= 0 || top <= 0 || top > E || !x || !router || !dense || !chosen || !chosen_w)
        return PS_ERR_BAD_ARGUMENT;
    if (groups < 0 || (groups > 1 && (E % groups || keep <= 0 || keep > groups))) return PS_ERR_BAD_ARGUMENT;
    if (shared_gate_w && !shared_gate) return PS_ERR_BAD_ARGUMENT;
    if (E > ps::MOE_MAX_EXPERTS) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((T + ps::MOE_WARPS - 1) / ps::MOE_WARPS), block(ps::MOE_WARPS * 32);
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::moe_route_kernel<float>, grid, block, 0, s, (const float*)x, x_stride,
                              (const float*)router, router_stride, (const float*)shared_gate_w, dense, chosen,
                              chosen_w, shared_gate, T, W, E, top, groups, keep);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::moe_route_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)x,
                              x_stride, (const __nv_bfloat16*)router, router_stride,
                              (const __nv_bfloat16*)shared_gate_w, dense, chosen, chosen_w, shared_gate, T, W, E, top,
                              groups, keep);
    return PS_ERR_UNSUPPORTED;
}

// gate_up [T, 2 * columns] (gates, then ups); dense float32 [T, E]; shared_gate float32 [T] (read for columns
// from E * F on); inner [T, columns].
PS_EXPORT int ps_moe_gate_mul(const void* gate_up, int gu_stride, const float* dense, const float* shared_gate,
                              void* inner, int inner_stride, int T, int columns, int E, int F, int dtype,
                              void* stream) {
    if (T <= 0 || columns <= 0) return PS_OK;
    if (!gate_up || !dense || !inner || E <= 0 || F <= 0 || columns < E * F) return PS_ERR_BAD_ARGUMENT;
    if (columns > E * F && !shared_gate) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)T * columns;
    const long long blocks = (total + 255) / 256;
    const dim3 grid((unsigned)(blocks < 4736 ? blocks : 4736));
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::moe_gate_mul_kernel<float>, grid, dim3(256), 0, s, (const float*)gate_up, gu_stride,
                              dense, shared_gate, (float*)inner, inner_stride, T, columns, E, F);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::moe_gate_mul_kernel<__nv_bfloat16>, grid, dim3(256), 0, s,
                              (const __nv_bfloat16*)gate_up, gu_stride, dense, shared_gate, (__nv_bfloat16*)inner,
                              inner_stride, T, columns, E, F);
    return PS_ERR_UNSUPPORTED;
}
