// RMS norm in groups, and the residual sums of a layer that norms what a sublayer returns.
//
// group_rms_norm, one CTA per row:  the row of H numbers is cut into `groups` equal consecutive runs; each run is
// divided by its own sqrt(mean(run^2) + eps); the whole is multiplied by `gain` (float32 [H]).  groups = 1 is the
// plain RMS norm.  The row is read in its own type (float32, or the compute type: a product's output), held in
// shared memory as float32, and written in the output's type; `rows` gathers (out[r] = norm(x[rows[r]])).  A row
// may be normed in place.
//
// post_norm_add, one CTA per token, all float32:  a sublayer has added its result into the zeroed row y; then
//     x <- x + group_rms_norm(y) * gain;   y <- 0 (ready for the next sublayer)
// and, where the layer ends with an average over depth (`history` given: [n][tokens][H], entries 0 .. n - 2 the
// embedding output and the results of the layers before, as they left this kernel):
//     history[n - 1] <- x;   x <- sum_j weight[j] * history[j]   (j rising)
// x is also left in the compute type (`x_cast`, null where that is float32 itself) for the next product.
//
// depth_begin: history[0] <- x (if given), x_cast <- x, y <- 0.
#include "common.cuh"

namespace ps {

constexpr int GROUP_NORM_THREADS = 256;
constexpr int GROUP_NORM_MAX_GROUPS = 64;

// sums of squares of the runs of the staged row -> 1 / sqrt(mean + eps) per run
__device__ __forceinline__ void group_inverse_rms(const float* staged, int H, int groups, float eps, float* inverse) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int run = H / groups;
    for (int g = warp; g < groups; g += warps) {
        const float* part = staged + (size_t)g * run;
        float sq = 0.f;
        for (int j = lane; j < run; j += 32) sq = fmaf(part[j], part[j], sq);
        sq = warp_sum(sq);
        if (lane == 0) inverse[g] = 1.0f / sqrtf(sq / (float)run + eps);
    }
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(GROUP_NORM_THREADS)
group_rms_norm_kernel(const TIn* x, long long x_stride, const int* __restrict__ rows, int H, int groups,
                      const float* __restrict__ gain, float eps, TOut* out, long long out_stride) {
    extern __shared__ float staged[];
    __shared__ float inverse[GROUP_NORM_MAX_GROUPS];
    pdl_prologue();
    x = pdl_fresh(x);
    const int r = blockIdx.x;
    const TIn* source = x + (size_t)(rows ? rows[r] : r) * x_stride;
    for (int j = threadIdx.x; j < H; j += blockDim.x) staged[j] = to_float(source[j]);
    __syncthreads();
    group_inverse_rms(staged, H, groups, eps, inverse);
    __syncthreads();
    const int run = H / groups;
    TOut* target = out + (size_t)r * out_stride;
    for (int j = threadIdx.x; j < H; j += blockDim.x) target[j] = from_float<TOut>(staged[j] * inverse[j / run] * gain[j]);
}

// V numbers per access (4 where the width allows it).  The older entries of the history do not depend on the
// sublayer's row: their weighted sum and the residual row are fetched in the first pass, beside the row itself, so
// that their latency lies behind the row's statistics instead of behind them.
template <int V> struct PackOf;
template <> struct PackOf<1> { float v[1]; };
template <> struct __align__(16) PackOf<4> { float v[4]; };

template <int V> __device__ __forceinline__ void store_cast(float* p, const PackOf<V>& a) { *reinterpret_cast<PackOf<V>*>(p) = a; }
template <int V> __device__ __forceinline__ void store_cast(__nv_bfloat16* p, const PackOf<V>& a) {
    if constexpr (V == 4) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a.v[0], a.v[1]), hi = __floats2bfloat162_rn(a.v[2], a.v[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = packed;
    } else {
        p[0] = __float2bfloat16_rn(a.v[0]);
    }
}

template <typename TC, int V>
__global__ void __launch_bounds__(GROUP_NORM_THREADS)
post_norm_add_kernel(float* __restrict__ y, float* __restrict__ x, int H, int groups, const float* __restrict__ gain,
                     float eps, TC* __restrict__ x_cast, float* history, long long history_stride,
                     int n_history, const float* __restrict__ weight) {
    using Pack = PackOf<V>;
    extern __shared__ __align__(16) float staged[];          // the sublayer's row, the residual row, the older entries' sum
    __shared__ float inverse[GROUP_NORM_MAX_GROUPS];
    float* row = staged;
    float* kept = staged + H;
    float* older = staged + 2 * H;
    pdl_prologue();
    y = pdl_fresh(y);
    x = pdl_fresh(x);
    history = pdl_fresh(history);
    const size_t base = (size_t)blockIdx.x * H;
    for (int j = V * threadIdx.x; j < H; j += V * blockDim.x) {
        const Pack a = *reinterpret_cast<const Pack*>(y + base + j);
        const Pack b = *reinterpret_cast<const Pack*>(x + base + j);
        Pack sum;
#pragma unroll
        for (int i = 0; i < V; ++i) sum.v[i] = 0.f;
        if (history) {
            for (int d = 0; d < n_history - 1; ++d) {
                const Pack h = *reinterpret_cast<const Pack*>(history + (size_t)d * history_stride + base + j);
                const float w = weight[d];
#pragma unroll
                for (int i = 0; i < V; ++i) sum.v[i] = fmaf(w, h.v[i], sum.v[i]);
            }
        }
        Pack zero;
#pragma unroll
        for (int i = 0; i < V; ++i) zero.v[i] = 0.f;
        *reinterpret_cast<Pack*>(y + base + j) = zero;
        *reinterpret_cast<Pack*>(row + j) = a;
        *reinterpret_cast<Pack*>(kept + j) = b;
        *reinterpret_cast<Pack*>(older + j) = sum;
    }
    __syncthreads();
    group_inverse_rms(row, H, groups, eps, inverse);
    __syncthreads();
    const int run = H / groups;
    const float newest = history ? weight[n_history - 1] : 1.f;
    for (int j = V * threadIdx.x; j < H; j += V * blockDim.x) {
        const Pack g = *reinterpret_cast<const Pack*>(gain + j);
        Pack v, out;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            v.v[i] = kept[j + i] + row[j + i] * inverse[(j + i) / run] * g.v[i];
            out.v[i] = history ? fmaf(newest, v.v[i], older[j + i]) : v.v[i];
        }
        if (history) *reinterpret_cast<Pack*>(history + (size_t)(n_history - 1) * history_stride + base + j) = v;
        *reinterpret_cast<Pack*>(x + base + j) = out;
        if (x_cast) store_cast<V>(x_cast + base + j, out);
    }
}

template <typename TC>
__global__ void __launch_bounds__(256)
depth_begin_kernel(const float* __restrict__ x, float* __restrict__ first, TC* __restrict__ x_cast, float* __restrict__ y,
                   long long count) {
    pdl_prologue();
    x = pdl_fresh(x);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const float v = x[i];
        if (first) first[i] = v;
        if (x_cast) x_cast[i] = from_float<TC>(v);
        y[i] = 0.f;
    }
}

template <typename TIn, typename TOut>
inline int launch_group_norm(const void* x, long long x_stride, const int* rows, int n_rows, int H, int groups,
                             const float* gain, float eps, void* out, long long out_stride, cudaStream_t s) {
    return launch_pdl(group_rms_norm_kernel<TIn, TOut>, dim3(n_rows), dim3(GROUP_NORM_THREADS), (size_t)H * sizeof(float),
                      s, (const TIn*)x, x_stride, rows, H, groups, gain, eps, (TOut*)out, out_stride);
}

}  // namespace ps

// x [*, H] rows of `in_dtype` with x_stride elements between rows; rows (may be null): int32 [n_rows] row indices;
// gain float32 [H]; out [n_rows, H] rows of `out_dtype`.  H must be a multiple of groups.
PS_EXPORT int ps_group_rms_norm(const void* x, long long x_stride, int in_dtype, const int* rows, int n_rows, int H,
                                int groups, const float* gain, float eps, void* out, long long out_stride,
                                int out_dtype, void* stream) {
    if (n_rows <= 0) return PS_OK;
    if (!x || !gain || !out || H <= 0 || groups <= 0 || H % groups) return PS_ERR_BAD_ARGUMENT;
    if (groups > ps::GROUP_NORM_MAX_GROUPS || (size_t)H * sizeof(float) > 48 * 1024) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define PS_GROUP_NORM(TIN, TOUT) \
    return ps::launch_group_norm<TIN, TOUT>(x, x_stride, rows, n_rows, H, groups, gain, eps, out, out_stride, s)
    if (in_dtype == PS_F32 && out_dtype == PS_F32) PS_GROUP_NORM(float, float);
    if (in_dtype == PS_F32 && out_dtype == PS_BF16) PS_GROUP_NORM(float, __nv_bfloat16);
    if (in_dtype == PS_BF16 && out_dtype == PS_BF16) PS_GROUP_NORM(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == PS_BF16 && out_dtype == PS_F32) PS_GROUP_NORM(__nv_bfloat16, float);
#undef PS_GROUP_NORM
    return PS_ERR_UNSUPPORTED;
}

// y, x float32 [T, H] contiguous; gain float32 [H]; x_cast [T, H] of `cast_dtype` or null; history float32
// [n_history][T][H] with history_stride elements between entries, or null; weight float32 [n_history].
PS_EXPORT int ps_post_norm_add(float* y, float* x, int T, int H, int groups, const float* gain, float eps, void* x_cast,
                               int cast_dtype, float* history, long long history_stride, int n_history,
                               const float* weight, void* stream) {
    if (T <= 0) return PS_OK;
    if (!y || !x || !gain || H <= 0 || groups <= 0 || H % groups) return PS_ERR_BAD_ARGUMENT;
    if (history && (!weight || n_history < 1)) return PS_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)3 * H * sizeof(float);
    if (groups > ps::GROUP_NORM_MAX_GROUPS || smem > 200 * 1024) return PS_ERR_UNSUPPORTED;
    if (x_cast && cast_dtype != PS_F32 && cast_dtype != PS_BF16) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const bool bf16 = x_cast && cast_dtype == PS_BF16;
    const bool by4 = H % 4 == 0 && history_stride % 4 == 0 &&
                     !(((uintptr_t)y | (uintptr_t)x | (uintptr_t)gain | (uintptr_t)history) & 15) &&
                     !((uintptr_t)x_cast & (bf16 ? 7 : 15));
#define PS_POST_NORM(TYPE, V)                                                                                        \
    do {                                                                                                             \
        static size_t raised[ps::MAX_DEVICES] = {0};                                                                 \
        auto kernel = ps::post_norm_add_kernel<TYPE, V>;                                                             \
        if (!ps::ensure_dynamic_smem((const void*)kernel, smem, raised)) return PS_ERR_LAUNCH;                       \
        return ps::launch_pdl(kernel, dim3(T), dim3(ps::GROUP_NORM_THREADS), smem, s, y, x, H, groups, gain, eps,    \
                              (TYPE*)x_cast, history, history_stride, n_history, weight);                            \
    } while (0)
    if (bf16) {
        if (by4) PS_POST_NORM(__nv_bfloat16, 4);
        PS_POST_NORM(__nv_bfloat16, 1);
    }
    if (by4) PS_POST_NORM(float, 4);
    PS_POST_NORM(float, 1);
#undef PS_POST_NORM
}

// x float32 [count]; first (may be null), y float32 [count]; x_cast [count] of `cast_dtype` or null.
PS_EXPORT int ps_depth_begin(const float* x, float* first, void* x_cast, int cast_dtype, float* y, long long count,
                             void* stream) {
    if (count <= 0) return PS_OK;
    if (!x || !y) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const long long blocks = (count + 255) / 256;
    const dim3 grid((unsigned)(blocks < 2368 ? blocks : 2368));
    if (!x_cast || cast_dtype == PS_F32)
        return ps::launch_pdl(ps::depth_begin_kernel<float>, grid, dim3(256), 0, s, x, first, (float*)x_cast, y, count);
    if (cast_dtype == PS_BF16)
        return ps::launch_pdl(ps::depth_begin_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, x, first, (__nv_bfloat16*)x_cast,
                              y, count);
    return PS_ERR_UNSUPPORTED;
}
