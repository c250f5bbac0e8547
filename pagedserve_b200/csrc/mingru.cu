// minGRU: a gated recurrence whose gates read only the current token.
//
// Per channel c of `width`, with the three projections of a token side by side in one float32 row
// [z' | u | g'] (biases already added by the product):
//     z = sigmoid(z');   candidate = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//     S_t = (1 - z_t) S_(t-1) + z_t candidate_t            (S: float32, one number per channel, kept in the slot)
//     out_t = S_t * silu(g'_t)                             (compute type: the output product's operand)
// An entry of the step runs its tokens in order from its request's stored S and leaves the new S there; an entry of
// one token is a decode step.  Everything is float32.
//
// The recurrence is linear in S, S_t = a_t S_(t-1) + b_t, so a long entry is cut into blockDim.y segments of
// consecutive tokens: every thread first folds its segment into one pair (A, B) = (prod a, the segment's result from
// zero), the pairs before a segment give its starting S, and a second pass over the segment writes the outputs.
// A CTA is blockDim.x channels of one entry; the second pass re-reads what the first has just brought into L2.
#include "common.cuh"

namespace ps {

constexpr int MINGRU_MAX_THREADS = 1024;
constexpr int MINGRU_AHEAD = 4;                 // tokens whose projections a thread has in flight

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename TC>
__global__ void __launch_bounds__(MINGRU_MAX_THREADS)
mingru_scan_kernel(const float* __restrict__ zug, long long row_stride, int width, float* __restrict__ state,
                   long long state_stride, const int* __restrict__ q_start, const int* __restrict__ item_slot,
                   TC* __restrict__ out, long long out_stride) {
    __shared__ float fold_a[MINGRU_MAX_THREADS];
    __shared__ float fold_b[MINGRU_MAX_THREADS];
    const int item = blockIdx.y;
    const int first = q_start[item], count = q_start[item + 1] - first;      // static for the step
    if (count <= 0) return;                                                   // (uniform over the CTA)
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = c < width;
    const int segments = blockDim.y, segment = threadIdx.y;
    const int per = (count + segments - 1) / segments;
    const int lo = min(segment * per, count), hi = min(lo + per, count);
    float* kept = state + (size_t)item_slot[item] * state_stride;
    pdl_prologue();
    zug = pdl_fresh(zug);
    float s = live ? kept[c] : 0.f;                    // every thread reads the stored S before anyone replaces it
    if (count == 1 && segments == 1) {                 // a decode step's entry: one token, straight through
        if (!live) return;
        const float* row = zug + (size_t)first * row_stride;
        const float z = sigmoid_f(row[c]);
        const float u = row[width + c];
        const float g = row[2 * width + c];
        const float candidate = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        s = (1.0f - z) * s + z * candidate;
        out[(size_t)first * out_stride + c] = from_float<TC>(s * (g / (1.0f + expf(-g))));
        kept[c] = s;
        return;
    }
    if (segments > 1) {
        float a_all = 1.f, b_all = 0.f;
        if (live) {
            // MINGRU_AHEAD tokens' gates are fetched before any of them is used: the loads do not depend on the fold
            for (int t0 = lo; t0 < hi; t0 += MINGRU_AHEAD) {
                float zs[MINGRU_AHEAD], us[MINGRU_AHEAD];
#pragma unroll
                for (int k = 0; k < MINGRU_AHEAD; ++k) {
                    const float* row = zug + (size_t)(first + min(t0 + k, hi - 1)) * row_stride;
                    zs[k] = row[c];
                    us[k] = row[width + c];
                }
#pragma unroll
                for (int k = 0; k < MINGRU_AHEAD; ++k) {
                    if (t0 + k >= hi) break;
                    const float z = sigmoid_f(zs[k]);
                    const float candidate = us[k] >= 0.f ? us[k] + 0.5f : sigmoid_f(us[k]);
                    const float a = 1.0f - z;
                    b_all = a * b_all + z * candidate;
                    a_all *= a;
                }
            }
        }
        fold_a[segment * blockDim.x + threadIdx.x] = a_all;
        fold_b[segment * blockDim.x + threadIdx.x] = b_all;
        __syncthreads();
        for (int before = 0; before < segment; ++before)
            s = fold_a[before * blockDim.x + threadIdx.x] * s + fold_b[before * blockDim.x + threadIdx.x];
    }
    if (!live) return;
    for (int t0 = lo; t0 < hi; t0 += MINGRU_AHEAD) {
        float zs[MINGRU_AHEAD], us[MINGRU_AHEAD], gs[MINGRU_AHEAD];
#pragma unroll
        for (int k = 0; k < MINGRU_AHEAD; ++k) {
            const float* row = zug + (size_t)(first + min(t0 + k, hi - 1)) * row_stride;
            zs[k] = row[c];
            us[k] = row[width + c];
            gs[k] = row[2 * width + c];
        }
#pragma unroll
        for (int k = 0; k < MINGRU_AHEAD; ++k) {
            if (t0 + k >= hi) break;
            const float z = sigmoid_f(zs[k]);
            const float candidate = us[k] >= 0.f ? us[k] + 0.5f : sigmoid_f(us[k]);
            s = (1.0f - z) * s + z * candidate;
            out[(size_t)(first + t0 + k) * out_stride + c] = from_float<TC>(s * (gs[k] / (1.0f + expf(-gs[k]))));
        }
    }
    if (hi == count && lo < hi) kept[c] = s;            // the segment that holds the entry's last token
}

}  // namespace ps

// zug float32 [T, 3 * width] rows (row_stride elements apart): z', u, g' side by side; state float32
// [slots, width] rows (state_stride apart); q_start int32 [items + 1]; item_slot int32 [items]; out [T, width] rows of
// `dtype`.  `segments` (1 .. 64): how many runs of consecutive tokens an entry is cut into.
PS_EXPORT int ps_mingru_scan(const float* zug, long long row_stride, int width, float* state, long long state_stride,
                             const int* q_start, const int* item_slot, int items, void* out, long long out_stride,
                             int segments, int dtype, void* stream) {
    if (items <= 0) return PS_OK;
    if (!zug || !state || !q_start || !item_slot || !out || width <= 0) return PS_ERR_BAD_ARGUMENT;
    if (segments < 1 || segments > 64) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    int channels = ps::MINGRU_MAX_THREADS / segments;
    if (channels > 128) channels = 128;
    while (channels > 32 && channels / 2 >= width) channels /= 2;
    // few entries of a narrow layer: fewer channels a CTA, so that the grid still covers the SMs
    while (channels > 8 && (long long)((width + channels - 1) / channels) * items < 148) channels /= 2;
    const dim3 grid((width + channels - 1) / channels, items), block(channels, segments);
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::mingru_scan_kernel<float>, grid, block, 0, s, zug, row_stride, width, state,
                              state_stride, q_start, item_slot, (float*)out, out_stride);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::mingru_scan_kernel<__nv_bfloat16>, grid, block, 0, s, zug, row_stride, width, state,
                              state_stride, q_start, item_slot, (__nv_bfloat16*)out, out_stride);
    return PS_ERR_UNSUPPORTED;
}
