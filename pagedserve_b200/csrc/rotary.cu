// Rotary position encoding fused with the cache write.
//
// One launch per attention layer and step, between the q|k(|v) projection and attention:
//   * queries are turned in place;
//   * keys are turned on their way into the key pages (the projection's buffer keeps them as projected);
//   * values go into the value pages: the rows of `v`, or, when `v` is null, the keys as projected
//     (a layer whose values are its unturned keys needs no value projection and no second buffer).
//
// The first rot_dims dimensions of every head turn, the rest pass. Pair i (i < rot_dims / 2) is
//   (2i, 2i + 1)             interleaved = 1
//   (i, i + rot_dims / 2)    interleaved = 0
// and (a, b) at position p becomes (a cos t - b sin t, b cos t + a sin t), t = p * inv_freq[i].
// Positions, angles, sines and products are float32 (inv_freq is a float32 table made on the host);
// results are rounded once to the storage type.
//
// Cache layout of one cache layer: pool[page * page_stride + (g * page_size + offset) * head_dim + d].
#include "common.cuh"

namespace ps {

constexpr int ROTARY_MAX_PAIRS = 256;

// two neighbouring elements as one access
template <typename T> struct PairOf;
template <> struct PairOf<float> { using type = float2; };
template <> struct PairOf<__nv_bfloat16> { using type = __nv_bfloat162; };
__device__ __forceinline__ float2 pair_to_float(float2 v) { return v; }
__device__ __forceinline__ float2 pair_to_float(__nv_bfloat162 v) { return __bfloat1622float2(v); }
template <typename P> __device__ __forceinline__ P pair_from_float(float a, float b);
template <> __device__ __forceinline__ float2 pair_from_float<float2>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 pair_from_float<__nv_bfloat162>(float a, float b) {
    return __floats2bfloat162_rn(a, b);
}                      // turning pairs of a head: head sizes up to 512

template <typename T>
__global__ void __launch_bounds__(256)
rotary_cache_write_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                          const T* __restrict__ v, int v_stride, const float* __restrict__ inv_freq, int rot_dims,
                          int interleaved, const int* __restrict__ token_row, const int* __restrict__ positions,
                          const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_pool,
                          T* __restrict__ v_pool, long long page_stride, int n_heads, int n_kv_heads, int head_dim,
                          int page_size) {
    pdl_prologue();
    q = pdl_fresh(q);
    k = pdl_fresh(k);
    v = pdl_fresh(v);
    const int t = blockIdx.x;
    const int p = positions[t];
    const int half = rot_dims >> 1;
    const int units = half + (head_dim - rot_dims);        // per head: turning pairs, then passing singles
    long long page_base = -1;
    if (k_pool) {
        const int page = block_table[(size_t)token_row[t] * bt_stride + p / page_size];
        if (page >= 0) page_base = (long long)page * page_stride + (long long)(p % page_size) * head_dim;
    }
    // a token's sines and cosines are the same for every head: once into shared memory
    __shared__ float2 turn[ROTARY_MAX_PAIRS];
    const float pos = (float)p;
    for (int unit = threadIdx.x; unit < half; unit += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[unit], &sn, &cs);
        turn[unit] = make_float2(cs, sn);
    }
    __syncthreads();
    T* q_row = q + (size_t)t * q_stride;
    const T* k_row = k + (size_t)t * k_stride;
    const int total = (n_heads + n_kv_heads) * units;
    // Neighbouring pairs, an even head size and even strides: every pair of a head, turning or not, is one access
    // of two elements (the addresses below are then multiples of the pair's size).
    using P = typename PairOf<T>::type;
    const bool by_pairs = interleaved && !(head_dim & 1) && !(q_stride & 1) && !(k_stride & 1) && !(v_stride & 1) &&
                          !(page_stride & 1) &&
                          !(((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)k_pool | (uintptr_t)v_pool) &
                            (sizeof(P) - 1));
    if (by_pairs) {
        const int pairs = head_dim >> 1;
        const int total_pairs = (n_heads + n_kv_heads) * pairs;
        for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < total_pairs; idx += gridDim.y * blockDim.x) {
            const int head = idx / pairs, u = idx - head * pairs;
            const bool turns = u < half;
            const float cs = turns ? turn[u].x : 1.f, sn = turns ? turn[u].y : 0.f;
            if (head < n_heads) {
                if (!turns) continue;
                P* at = reinterpret_cast<P*>(q_row + head * head_dim) + u;
                const float2 ab = pair_to_float(*at);
                *at = pair_from_float<P>(ab.x * cs - ab.y * sn, ab.y * cs + ab.x * sn);
            } else if (page_base >= 0) {
                const int g = head - n_heads;
                const P key = reinterpret_cast<const P*>(k_row + g * head_dim)[u];
                const long long dst = page_base + (long long)g * page_size * head_dim + 2 * u;
                P turned = key;
                if (turns) {
                    const float2 ab = pair_to_float(key);
                    turned = pair_from_float<P>(ab.x * cs - ab.y * sn, ab.y * cs + ab.x * sn);
                }
                *reinterpret_cast<P*>(k_pool + dst) = turned;
                *reinterpret_cast<P*>(v_pool + dst) =
                    v ? reinterpret_cast<const P*>(v + (size_t)t * v_stride + g * head_dim)[u] : key;
            }
        }
        return;
    }
    // few tokens (decode): the heads of a token are shared out over gridDim.y CTAs, one unit per thread
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < total; idx += gridDim.y * blockDim.x) {
        const int head = idx / units, unit = idx - head * units;
        const bool is_query = head < n_heads;
        const int g = head - n_heads;                      // key/value head when not a query
        if (unit >= half) {                                // a dimension that does not turn
            if (is_query || page_base < 0) continue;
            const int d = rot_dims + (unit - half);
            const T key = k_row[g * head_dim + d];
            const long long dst = page_base + (long long)g * page_size * head_dim + d;
            k_pool[dst] = key;
            v_pool[dst] = v ? v[(size_t)t * v_stride + g * head_dim + d] : key;
            continue;
        }
        const int da = interleaved ? 2 * unit : unit, db = interleaved ? 2 * unit + 1 : unit + half;
        const float cs = turn[unit].x, sn = turn[unit].y;
        if (is_query) {
            T* row = q_row + head * head_dim;
            const float a = to_float(row[da]), b = to_float(row[db]);
            row[da] = from_float<T>(a * cs - b * sn);
            row[db] = from_float<T>(b * cs + a * sn);
        } else if (page_base >= 0) {
            const T* row = k_row + g * head_dim;
            const T ka = row[da], kb = row[db];
            const float a = to_float(ka), b = to_float(kb);
            const long long dst = page_base + (long long)g * page_size * head_dim;
            k_pool[dst + da] = from_float<T>(a * cs - b * sn);
            k_pool[dst + db] = from_float<T>(b * cs + a * sn);
            if (v) {
                const T* vr = v + (size_t)t * v_stride + g * head_dim;
                v_pool[dst + da] = vr[da];
                v_pool[dst + db] = vr[db];
            } else {
                v_pool[dst + da] = ka;
                v_pool[dst + db] = kb;
            }
        }
    }
}


// ---- the same step for heads that are normed before they turn ----
// Per head, over its first `dim` numbers (a head occupies `head_dim` >= dim numbers of its row; what lies behind
// `dim` is padding and is carried along unchanged):
//     y = x / sqrt(mean(x^2) + eps) * gain          (gain float32 [dim], one for all query heads, one for all key
//                                                    heads; a null gain: no norm)
// then the first rot_dims numbers turn as above and the result goes back into q (queries) or into the key pages
// (keys); the rows of v go into the value pages as they are.  k null: a layer that reads keys and values that
// another layer cached; only its queries are prepared.  The angle p * f is formed to more than one float:
// every frequency comes as (high, low) parts, the product's rounding error is recovered with an fma and what the
// float that sincosf takes cannot hold is applied to first order.  Norm statistics, angles and products: float32.
// One warp per head; a token's heads are shared out over gridDim.y CTAs.
constexpr int HEAD_NORM_WARPS = 4;
constexpr int HEAD_NORM_MAX_DIM = 256;

template <typename T>
__global__ void __launch_bounds__(HEAD_NORM_WARPS * 32)
head_norm_rotary_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                        const T* __restrict__ v, int v_stride, const float* __restrict__ q_gain,
                        const float* __restrict__ k_gain, float eps, const float2* __restrict__ inv_freq, int rot_dims,
                        int interleaved, const int* __restrict__ token_row, const int* __restrict__ positions,
                        const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_pool,
                        T* __restrict__ v_pool, long long page_stride, int n_heads, int n_kv_heads, int head_dim,
                        int dim, int page_size, float amplitude) {
    __shared__ float2 turn[ROTARY_MAX_PAIRS];
    __shared__ float staged[HEAD_NORM_WARPS][HEAD_NORM_MAX_DIM];
    const int t = blockIdx.x;
    const int p = positions[t];                              // static for the step: read before the wait
    const int half = rot_dims >> 1;
    const float pos = (float)p;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float2 f = inv_freq[i];
        const float high = pos * f.x;
        const float low = fmaf(pos, f.x, -high) + pos * f.y;
        float sn, cs;
        sincosf(high, &sn, &cs);
        turn[i] = make_float2(fmaf(-low, sn, cs) * amplitude, fmaf(low, cs, sn) * amplitude);
    }
    pdl_prologue();
    q = pdl_fresh(q);
    k = pdl_fresh(k);
    v = pdl_fresh(v);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_heads = n_heads + (k ? n_kv_heads : 0);
    long long page_base = -1;
    if (k && k_pool) {
        const int page = block_table[(size_t)token_row[t] * bt_stride + p / page_size];
        if (page >= 0) page_base = (long long)page * page_stride + (long long)(p % page_size) * head_dim;
    }
    float* mine = staged[warp];
    for (int head = blockIdx.y * HEAD_NORM_WARPS + warp; head < total_heads; head += gridDim.y * HEAD_NORM_WARPS) {
        const bool is_query = head < n_heads;
        const int g = head - n_heads;
        const T* src = is_query ? q + (size_t)t * q_stride + (size_t)head * head_dim
                                : k + (size_t)t * k_stride + (size_t)g * head_dim;
        const float* gain = is_query ? q_gain : k_gain;
        float sq = 0.f;
        for (int d = lane; d < dim; d += 32) {
            const float x = to_float(src[d]);
            mine[d] = x;
            sq = fmaf(x, x, sq);
        }
        sq = warp_sum(sq);
        const float inv = gain ? 1.0f / sqrtf(sq / (float)dim + eps) : 1.0f;
        __syncwarp();
        if (gain)
            for (int d = lane; d < dim; d += 32) mine[d] = mine[d] * inv * gain[d];
        __syncwarp();
        T* dst = nullptr;
        if (is_query) dst = q + (size_t)t * q_stride + (size_t)head * head_dim;
        else if (page_base >= 0) dst = k_pool + page_base + (long long)g * page_size * head_dim;
        if (dst) {
            for (int unit = lane; unit < half; unit += 32) {
                const int da = interleaved ? 2 * unit : unit, db = interleaved ? 2 * unit + 1 : unit + half;
                const float a = mine[da], b = mine[db];
                const float cs = turn[unit].x, sn = turn[unit].y;
                dst[da] = from_float<T>(a * cs - b * sn);
                dst[db] = from_float<T>(b * cs + a * sn);
            }
            for (int d = rot_dims + lane; d < dim; d += 32) dst[d] = from_float<T>(mine[d]);
            if (!is_query) {
                for (int d = dim + lane; d < head_dim; d += 32) dst[d] = src[d];
                if (v) {
                    const T* value = v + (size_t)t * v_stride + (size_t)g * head_dim;
                    T* value_dst = v_pool + page_base + (long long)g * page_size * head_dim;
                    for (int d = lane; d < head_dim; d += 32) value_dst[d] = value[d];
                }
            }
        }
        __syncwarp();
    }
}


// The same step with four neighbouring numbers per access, for head sizes, strides and addresses that are multiples
// of four elements.  A head is worked on by `lanes` lanes of a warp (a power of two, at least head_dim / 8 up to 32:
// a warp takes several heads at once unless a head has more than 128 numbers), each lane holding two groups of four
// numbers, `4 * lanes` apart, whose loads are issued together (twice the bytes in flight of one group a lane); the
// sum of squares is reduced inside the head's lanes.  Neighbours paired: both numbers of a pair are in one lane.
// Halves paired: normed numbers pass through shared memory, written and (when a half is a multiple of four) read a
// quad per access, which keeps the banks free of conflicts; scalar accesses of stride four were what bounded this
// kernel before.  Every result leaves as one access of four.  Queries, keys and values are separate units of work:
// a token has n_heads + 2 * n_kv_heads of them (values are copied).  The gains are read by quads too: dim is a
// multiple of four and the gain tables start on 16-byte boundaries (the launcher checks).
template <typename T> struct QuadOf;
template <> struct QuadOf<float> { using type = float4; };
template <> struct QuadOf<__nv_bfloat16> { using type = uint2; };
__device__ __forceinline__ void quad_to_float(const float4& v, float (&x)[4]) { x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w; }
__device__ __forceinline__ void quad_to_float(const uint2& v, float (&x)[4]) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
__device__ __forceinline__ void quad_from_float(const float (&x)[4], float4& v) { v = make_float4(x[0], x[1], x[2], x[3]); }
__device__ __forceinline__ void quad_from_float(const float (&x)[4], uint2& v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    v.x = *reinterpret_cast<const uint32_t*>(&a);
    v.y = *reinterpret_cast<const uint32_t*>(&b);
}

// PAIRING is a template parameter so that a pass carries the code of its own form only: 0 neighbours paired, 1 halves
// paired with a half that is a multiple of four, 2 halves paired with any even number of turning dimensions.
template <typename T, int PAIRING>
__global__ void __launch_bounds__(HEAD_NORM_WARPS * 32, 16)
head_norm_rotary_quads_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                              const T* __restrict__ v, int v_stride, const float* __restrict__ q_gain,
                              const float* __restrict__ k_gain, float eps, const float2* __restrict__ inv_freq,
                              int rot_dims, const int* __restrict__ token_row,
                              const int* __restrict__ positions, const int* __restrict__ block_table, int bt_stride,
                              T* __restrict__ k_pool, T* __restrict__ v_pool, long long page_stride, int n_heads,
                              int n_kv_heads, int head_dim, int dim, int page_size, int lanes, float amplitude) {
    using Q = typename QuadOf<T>::type;
    constexpr bool interleaved = PAIRING == 0;
    __shared__ __align__(16) float2 turn[ROTARY_MAX_PAIRS];
    __shared__ __align__(16) float staged[HEAD_NORM_WARPS][HEAD_NORM_MAX_DIM];
    const int t = blockIdx.x;
    // positions, rows and the block table are static for the step: read before the wait
    const int p = positions[t];
    long long page_base = -1;
    if (k && k_pool) {
        const int page = block_table[(size_t)token_row[t] * bt_stride + p / page_size];
        if (page >= 0) page_base = (long long)page * page_stride + (long long)(p % page_size) * head_dim;
    }
    const int half = rot_dims >> 1;
    const float pos = (float)p;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float2 f = inv_freq[i];
        const float high = pos * f.x;
        const float low = fmaf(pos, f.x, -high) + pos * f.y;
        float sn, cs;
        sincosf(high, &sn, &cs);
        turn[i] = make_float2(fmaf(-low, sn, cs) * amplitude, fmaf(low, cs, sn) * amplitude);
    }
    pdl_prologue();
    q = pdl_fresh(q);
    k = pdl_fresh(k);
    v = pdl_fresh(v);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_warp = 32 / lanes, group = lane / lanes, gl = lane - group * lanes;
    const int kv = k ? n_kv_heads : 0;
    const int total = n_heads + 2 * kv;
    float* mine = staged[warp] + group * (lanes * 8);       // a head has at most 8 * lanes numbers
    const int step = gridDim.y * HEAD_NORM_WARPS * per_warp;
    for (int base = (blockIdx.y * HEAD_NORM_WARPS + warp) * per_warp; base < total; base += step) {
        // where this unit of work reads and writes: queries in place, keys and values from their rows into the pages
        const int unit = base + group;
        const bool is_query = unit < n_heads, is_value = unit >= n_heads + kv;
        const T* src = nullptr;
        T* dst = nullptr;
        if (unit < total) {
            if (is_query) {
                dst = q + (size_t)t * q_stride + (size_t)unit * head_dim;
                src = dst;
            } else {
                const int g = is_value ? unit - n_heads - kv : unit - n_heads;
                src = (is_value ? v + (size_t)t * v_stride : k + (size_t)t * k_stride) + (size_t)g * head_dim;
                if (page_base >= 0) dst = (is_value ? v_pool : k_pool) + page_base + (long long)g * page_size * head_dim;
            }
        }
        float x[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int d0 = (gl + j * lanes) * 4;
            if (dst && d0 < head_dim) {
                const Q raw = *reinterpret_cast<const Q*>(src + d0);
                if (is_value) *reinterpret_cast<Q*>(dst + d0) = raw;          // values go straight to their page
                else quad_to_float(raw, x[j]);
            }
        }
        const bool turns = dst && !is_value;
        const float* gain = is_query ? q_gain : k_gain;
        float sq = 0.f;
        if (turns) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int d0 = (gl + j * lanes) * 4;
                if (d0 < dim) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) sq = fmaf(x[j][e], x[j][e], sq);
                }
            }
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float inv = gain ? 1.0f / sqrtf(sq / (float)dim + eps) : 1.0f;
        if (turns) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int d0 = (gl + j * lanes) * 4;
                if (d0 < head_dim) {
                    if (gain && d0 < dim) {
                        const float4 w = *reinterpret_cast<const float4*>(gain + d0);
                        x[j][0] = x[j][0] * inv * w.x;
                        x[j][1] = x[j][1] * inv * w.y;
                        x[j][2] = x[j][2] * inv * w.z;
                        x[j][3] = x[j][3] * inv * w.w;
                    }
                    // partners in another quad: the normed numbers pass through shared memory, a quad per access
                    if constexpr (!interleaved) *reinterpret_cast<float4*>(mine + d0) = make_float4(x[j][0], x[j][1], x[j][2], x[j][3]);
                }
            }
        }
        __syncwarp();
        if (turns) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int d0 = (gl + j * lanes) * 4;
                if (d0 < head_dim) {
                    float y[4] = {x[j][0], x[j][1], x[j][2], x[j][3]};
                    if (d0 < rot_dims) {
                        if constexpr (interleaved) {
                            // both pairs of the quad are in this lane's registers; rot_dims is even, so a quad
                            // holds two turning pairs or, at the end, one
                            const float2 t0 = turn[d0 >> 1];
                            y[0] = x[j][0] * t0.x - x[j][1] * t0.y;
                            y[1] = x[j][1] * t0.x + x[j][0] * t0.y;
                            if (d0 + 2 < rot_dims) {
                                const float2 t1 = turn[(d0 >> 1) + 1];
                                y[2] = x[j][2] * t1.x - x[j][3] * t1.y;
                                y[3] = x[j][3] * t1.x + x[j][2] * t1.y;
                            }
                        } else if constexpr (PAIRING == 1) {
                            // halves of a multiple of four: the partner quad and its four (cos, sin) in whole accesses
                            const bool first = d0 < half;
                            const int pair = first ? d0 : d0 - half;
                            const float4 o = *reinterpret_cast<const float4*>(mine + (first ? d0 + half : d0 - half));
                            const float4 ta = *reinterpret_cast<const float4*>(&turn[pair]);
                            const float4 tb = *reinterpret_cast<const float4*>(&turn[pair + 2]);
                            const float sign = first ? -1.f : 1.f;
                            y[0] = fmaf(sign * o.x, ta.y, x[j][0] * ta.x);
                            y[1] = fmaf(sign * o.y, ta.w, x[j][1] * ta.z);
                            y[2] = fmaf(sign * o.z, tb.y, x[j][2] * tb.x);
                            y[3] = fmaf(sign * o.w, tb.w, x[j][3] * tb.z);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int d = d0 + e;
                                if (d < rot_dims) {
                                    const bool first = d < half;
                                    const float2 cs_sn = turn[first ? d : d - half];
                                    const float o = mine[first ? d + half : d - half];
                                    y[e] = first ? x[j][e] * cs_sn.x - o * cs_sn.y : x[j][e] * cs_sn.x + o * cs_sn.y;
                                }
                            }
                        }
                    }
                    Q packed;
                    quad_from_float(y, packed);
                    *reinterpret_cast<Q*>(dst + d0) = packed;
                }
            }
        }
        __syncwarp();
    }
}

}  // namespace ps

// Heads that are normed, then turned (see head_norm_rotary_kernel).  q [T, n_heads * head_dim] in place; k, v
// [T, n_kv_heads * head_dim] or both null (queries only); q_gain / k_gain float32 [dim] or null; inv_freq float32
// [rot_dims / 2][2] as (high, low) parts; k_pool null: nothing is written to pages.  `amplitude` multiplies every sine
// and cosine (1: a plain turn).
PS_EXPORT int ps_head_norm_rotary_cache_write(void* q, int q_stride, const void* k, int k_stride, const void* v,
                                              int v_stride, const float* q_gain, const float* k_gain, float eps,
                                              const float* inv_freq, int rot_dims, int interleaved,
                                              const int* token_row, const int* positions, const int* block_table,
                                              int bt_stride, void* k_pool, void* v_pool, long long page_stride, int T,
                                              int n_heads, int n_kv_heads, int head_dim, int dim, int page_size,
                                              int dtype, float amplitude, void* stream) {
    if (T <= 0) return PS_OK;
    if (n_heads <= 0 || n_kv_heads < 0 || head_dim <= 0 || dim <= 0 || dim > head_dim || rot_dims < 0 ||
        rot_dims > dim || (rot_dims & 1))
        return PS_ERR_BAD_ARGUMENT;
    if (rot_dims > 0 && (!inv_freq || ((uintptr_t)inv_freq & 7))) return PS_ERR_BAD_ARGUMENT;
    if (rot_dims / 2 > ps::ROTARY_MAX_PAIRS || dim > ps::HEAD_NORM_MAX_DIM) return PS_ERR_UNSUPPORTED;
    if (!positions || !q || (k && !v) || (!k && v)) return PS_ERR_BAD_ARGUMENT;
    if (k && k_pool && (!v_pool || !token_row || !block_table || page_size <= 0)) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int elem = dtype == PS_F32 ? 4 : 2;
    const uintptr_t addresses = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)k_pool | (uintptr_t)v_pool;
    const bool gains_by_quads = !(dim & 3) && !(((uintptr_t)q_gain | (uintptr_t)k_gain) & 15);
    const bool quads = gains_by_quads && head_dim <= ps::HEAD_NORM_MAX_DIM && !(head_dim & 3) && !(q_stride & 3) && !(k_stride & 3) && !(v_stride & 3) && !(page_stride & 3) &&
                       !(addresses & (uintptr_t)(4 * elem - 1));
    if (quads && (dtype == PS_F32 || dtype == PS_BF16)) {
        int lanes = 1;
        while (lanes < 32 && lanes * 8 < head_dim) lanes <<= 1;    // two quads a lane: both loads in flight at once
        const int units = n_heads + (k ? 2 * n_kv_heads : 0);
        const int per_cta = ps::HEAD_NORM_WARPS * (32 / lanes);
        int split = (units + per_cta - 1) / per_cta;
        if (T >= 2048 && split > 2) split = 2;               // many tokens: fewer CTAs, each walks several heads
        const dim3 grid(T, split), block(ps::HEAD_NORM_WARPS * 32);
        const int pairing = interleaved ? 0 : (((rot_dims >> 1) & 3) ? 2 : 1);
#define PS_HEAD_NORM_QUADS(TYPE, PAIRING)                                                                              \
    ps::launch_pdl(ps::head_norm_rotary_quads_kernel<TYPE, PAIRING>, grid, block, 0, s, (TYPE*)q, q_stride,             \
                   (const TYPE*)k, k_stride, (const TYPE*)v, v_stride, q_gain, k_gain, eps, (const float2*)inv_freq,   \
                   rot_dims, token_row, positions, block_table, bt_stride, (TYPE*)k_pool, (TYPE*)v_pool, page_stride,  \
                   n_heads, n_kv_heads, head_dim, dim, page_size, lanes, amplitude)
        if (dtype == PS_F32)
            return pairing == 0 ? PS_HEAD_NORM_QUADS(float, 0)
                                : pairing == 1 ? PS_HEAD_NORM_QUADS(float, 1) : PS_HEAD_NORM_QUADS(float, 2);
        return pairing == 0 ? PS_HEAD_NORM_QUADS(__nv_bfloat16, 0)
                            : pairing == 1 ? PS_HEAD_NORM_QUADS(__nv_bfloat16, 1) : PS_HEAD_NORM_QUADS(__nv_bfloat16, 2);
#undef PS_HEAD_NORM_QUADS
    }
    const int heads = n_heads + (k ? n_kv_heads : 0);
    int split = (heads + ps::HEAD_NORM_WARPS - 1) / ps::HEAD_NORM_WARPS;
    if (T >= 2048 && split > 2) split = 2;                   // many tokens: fewer CTAs, each walks several heads
    const dim3 grid(T, split), block(ps::HEAD_NORM_WARPS * 32);
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::head_norm_rotary_kernel<float>, grid, block, 0, s, (float*)q, q_stride,
                              (const float*)k, k_stride, (const float*)v, v_stride, q_gain, k_gain, eps,
                              (const float2*)inv_freq, rot_dims, interleaved, token_row, positions, block_table,
                              bt_stride, (float*)k_pool, (float*)v_pool, page_stride, n_heads, n_kv_heads, head_dim,
                              dim, page_size, amplitude);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::head_norm_rotary_kernel<__nv_bfloat16>, grid, block, 0, s, (__nv_bfloat16*)q,
                              q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, q_gain,
                              k_gain, eps, (const float2*)inv_freq, rot_dims, interleaved, token_row, positions,
                              block_table, bt_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride,
                              n_heads, n_kv_heads, head_dim, dim, page_size, amplitude);
    return PS_ERR_UNSUPPORTED;
}

// q [T, n_heads * head_dim] is turned in place. k [T, n_kv_heads * head_dim] is read only. v may be null: the
// values are then the keys as projected. k_pool null: nothing is written to pages (queries only).
PS_EXPORT int ps_rotary_cache_write(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                                    const float* inv_freq, int rot_dims, int interleaved, const int* token_row,
                                    const int* positions, const int* block_table, int bt_stride, void* k_pool,
                                    void* v_pool, long long page_stride, int T, int n_heads, int n_kv_heads,
                                    int head_dim, int page_size, int dtype, void* stream) {
    if (T <= 0) return PS_OK;
    if (n_heads < 0 || n_kv_heads < 0 || head_dim <= 0 || rot_dims < 0 || rot_dims > head_dim || (rot_dims & 1))
        return PS_ERR_BAD_ARGUMENT;
    if (rot_dims > 0 && !inv_freq) return PS_ERR_BAD_ARGUMENT;
    if (rot_dims / 2 > ps::ROTARY_MAX_PAIRS) return PS_ERR_UNSUPPORTED;
    if (k_pool && (!v_pool || !token_row || !block_table || page_size <= 0)) return PS_ERR_BAD_ARGUMENT;
    if (!positions || !q || !k) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int work = (n_heads + n_kv_heads) * (rot_dims / 2 + head_dim - rot_dims);
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    // a step of few tokens is bound by the chain of loads of one thread: spread a token over several CTAs
    const int split = T >= 512 ? 1 : (work + threads - 1) / threads;
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::rotary_cache_write_kernel<float>, dim3(T, split), dim3(threads), 0, s, (float*)q, q_stride,
                              (const float*)k, k_stride, (const float*)v, v_stride, inv_freq, rot_dims, interleaved,
                              token_row, positions, block_table, bt_stride, (float*)k_pool, (float*)v_pool,
                              page_stride, n_heads, n_kv_heads, head_dim, page_size);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::rotary_cache_write_kernel<__nv_bfloat16>, dim3(T, split), dim3(threads), 0, s,
                              (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride,
                              (const __nv_bfloat16*)v, v_stride, inv_freq, rot_dims, interleaved, token_row, positions,
                              block_table, bt_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride,
                              n_heads, n_kv_heads, head_dim, page_size);
    return PS_ERR_UNSUPPORTED;
}
