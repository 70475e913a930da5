// Several residual streams with learned mixing ("hyper-connections").
//
// Instead of one residual row x per token there are S rows x_1 .. x_S.  A sublayer f with the weights
// in[S], out[S], mix[S, S] (mix indexed [from, to]) does
//     u    = sum_s in[s] x_s
//     y    = f(norm(u))
//     x_t <- sum_s mix[s, t] x_s + out[t] y        (all t from the old rows)
// Everything is float32.  The streams of a step are one array [S, T, W].
//
// hyper_begin:  x_s = x0 for every s, u = sum_s in[s] x_s, y = 0.
// hyper_step:   finishes one sublayer and opens the next in one pass over the streams: the update above with the
//               finished sublayer's (mix, out, y), then u = sum_t in_next[t] x_t with the next sublayer's weights
//               (ones at the end of the model: u is then the sum of the streams), then y = 0 for the next
//               sublayer to add its result into.
// Sums run over s in rising order.
#include "common.cuh"

namespace ps {

constexpr int HYPER_MAX_STREAMS = 8;

__global__ void __launch_bounds__(256)
hyper_begin_kernel(const float* __restrict__ x0, const float* __restrict__ in, float* __restrict__ streams,
                   float* __restrict__ u, float* __restrict__ y, long long count, int S) {
    pdl_prologue();
    x0 = pdl_fresh(x0);
    float w[HYPER_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HYPER_MAX_STREAMS; ++s) w[s] = s < S ? in[s] : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        const float x = x0[i];
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
            if (s < S) {
                streams[(long long)s * count + i] = x;
                acc = s == 0 ? w[0] * x : acc + w[s] * x;
            }
        u[i] = acc;
        y[i] = 0.f;
    }
}

__global__ void __launch_bounds__(256)
hyper_step_kernel(float* __restrict__ streams, float* __restrict__ y, const float* __restrict__ mix,
                  const float* __restrict__ out, const float* __restrict__ in_next, float* __restrict__ u,
                  long long count, int S) {
    __shared__ float m[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS], o[HYPER_MAX_STREAMS], n[HYPER_MAX_STREAMS];
    if (threadIdx.x < S * S) m[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        o[threadIdx.x] = out[threadIdx.x];
        n[threadIdx.x] = in_next ? in_next[threadIdx.x] : 1.f;
    }
    __syncthreads();
    pdl_prologue();
    streams = pdl_fresh(streams);
    y = pdl_fresh(y);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        float x[HYPER_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HYPER_MAX_STREAMS; ++s) x[s] = s < S ? streams[(long long)s * count + i] : 0.f;
        const float f = y[i];
        float next = 0.f;
#pragma unroll
        for (int t = 0; t < HYPER_MAX_STREAMS; ++t)
            if (t < S) {
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
                    if (s < S) acc = s == 0 ? m[t] * x[0] : acc + m[s * S + t] * x[s];
                acc += o[t] * f;
                streams[(long long)t * count + i] = acc;
                next = t == 0 ? n[0] * acc : next + n[t] * acc;
            }
        u[i] = next;
        y[i] = 0.f;
    }
}

}  // namespace ps

// x0, u, y: float32 [count]; streams: float32 [S, count]; in: float32 [S].
PS_EXPORT int ps_hyper_begin(const float* x0, const float* in, float* streams, float* u, float* y, long long count,
                             int S, void* stream) {
    if (count <= 0) return PS_OK;
    if (S <= 0 || S > ps::HYPER_MAX_STREAMS) return PS_ERR_UNSUPPORTED;
    if (!x0 || !in || !streams || !u || !y) return PS_ERR_BAD_ARGUMENT;
    const long long blocks = (count + 255) / 256;
    return ps::launch_pdl(ps::hyper_begin_kernel, dim3((unsigned)(blocks < 4736 ? blocks : 4736)), dim3(256), 0,
                          (cudaStream_t)stream, x0, in, streams, u, y, count, S);
}

// mix: float32 [S, S] indexed [from, to]; out: float32 [S]; in_next: float32 [S] or null (ones).
PS_EXPORT int ps_hyper_step(float* streams, float* y, const float* mix, const float* out, const float* in_next,
                            float* u, long long count, int S, void* stream) {
    if (count <= 0) return PS_OK;
    if (S <= 0 || S > ps::HYPER_MAX_STREAMS) return PS_ERR_UNSUPPORTED;
    if (!streams || !y || !mix || !out || !u) return PS_ERR_BAD_ARGUMENT;
    const long long blocks = (count + 255) / 256;
    return ps::launch_pdl(ps::hyper_step_kernel, dim3((unsigned)(blocks < 4736 ? blocks : 4736)), dim3(256), 0,
                          (cudaStream_t)stream, streams, y, mix, out, in_next, u, count, S);
}
