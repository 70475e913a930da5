// Token embedding with a scale and a hashed table of token pairs.
//
//   h[t] = scale * table[id_t] + pair[row_t]
//   row_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets     for a token that has one before it,
//   row_t = buckets (the table's extra last row)                   for the first token of a sequence.
//
// The token before the first token of an entry is not in the step: it is the request's newest token of the
// step before, kept in the request's slot (one int32 per slot).  The CTA of an entry's first token reads that
// word and then stores the entry's last token there, so nothing else in the launch touches it.
// The sum is float32 (it starts the residual stream).
#include "common.cuh"

namespace ps {

template <typename T>
__global__ void embed_pair_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                  const int* __restrict__ token_item, const int* __restrict__ q_start,
                                  const int* __restrict__ item_slot, const T* __restrict__ table, float scale,
                                  const T* __restrict__ pair, int buckets, unsigned long long mul_prev,
                                  unsigned long long mul_cur, int* __restrict__ newest, float* __restrict__ out,
                                  int H, int V, int* __restrict__ status) {
    pdl_prologue();
    ids = pdl_fresh(ids);
    positions = pdl_fresh(positions);
    token_item = pdl_fresh(token_item);
    __shared__ int row_shared;
    const int t = blockIdx.x;
    const int id = ids[t];
    if (threadIdx.x == 0) {
        int row = -1;
        if (pair) {
            const int item = token_item[t];
            const int first = q_start[item];
            const int slot = item_slot[item];
            int before = -1;
            if (t > first) before = ids[t - 1];
            else if (positions[t] > 0) before = newest[slot];
            if (t == first) newest[slot] = ids[q_start[item + 1] - 1];
            if (positions[t] == 0) row = buckets;
            else if (before >= 0 && before < V && id >= 0)
                row = (int)((((unsigned long long)before % buckets) * mul_prev +
                             ((unsigned long long)id % buckets) * mul_cur) % (unsigned long long)buckets);
            else row = -2;
        }
        row_shared = row;
    }
    __syncthreads();
    const int row = row_shared;
    if (id < 0 || id >= V || row == -2) {
        if (threadIdx.x == 0 && status) atomicExch(status, 1);
        for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)t * H + c] = 0.f;
        return;
    }
    const T* e = table + (size_t)id * H;
    const T* b = row >= 0 ? pair + (size_t)row * H : nullptr;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = to_float(e[c]) * scale;
        if (b) v += to_float(b[c]);
        out[(size_t)t * H + c] = v;
    }
}

}  // namespace ps

// ids, positions, token_item [T]; q_start [items + 1]; item_slot [items]; table [V, H]; pair [buckets + 1, H] or
// null (no pair table: newest is not touched); mul_prev, mul_cur already reduced modulo buckets; newest: one int32
// per slot; out float32 [T, H].
PS_EXPORT int ps_embed_pair(const int* ids, const int* positions, const int* token_item, const int* q_start,
                            const int* item_slot, const void* table, float scale, const void* pair, int buckets,
                            long long mul_prev, long long mul_cur, int* newest, float* out, int T, int H, int V,
                            int dtype, int* status, void* stream) {
    if (T <= 0) return PS_OK;
    if (H <= 0 || V <= 0 || !ids || !table || !out) return PS_ERR_BAD_ARGUMENT;
    if (pair && (buckets <= 0 || mul_prev < 0 || mul_cur < 0 || mul_prev >= buckets || mul_cur >= buckets ||
                 !newest || !positions || !token_item || !q_start || !item_slot))
        return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = H >= 256 ? 256 : 128;
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::embed_pair_kernel<float>, dim3(T), dim3(nt), 0, s, ids, positions, token_item,
                              q_start, item_slot, (const float*)table, scale, (const float*)pair, buckets,
                              (unsigned long long)mul_prev, (unsigned long long)mul_cur, newest, out, H, V, status);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::embed_pair_kernel<__nv_bfloat16>, dim3(T), dim3(nt), 0, s, ids, positions,
                              token_item, q_start, item_slot, (const __nv_bfloat16*)table, scale,
                              (const __nv_bfloat16*)pair, buckets, (unsigned long long)mul_prev,
                              (unsigned long long)mul_cur, newest, out, H, V, status);
    return PS_ERR_UNSUPPORTED;
}
