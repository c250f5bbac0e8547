// Latent attention: what lies between the stacked input projection and attention, and the output gate.
//
// A token's keys and values of all heads are made from one small vector c (size R) and one turning key part
// (size r) shared by all heads, and only those two are cached:
//     c      = rms_norm(down[0:R]) * gain           down = W_dkv h, R + r numbers
//     k_turn = turn(down[R:R + r], p)
//     score(h) = (q_flat(h) . W_uk(h) c  +  turn(q_turn(h), p) . k_turn) * scale
//              = ([W_uk(h)^T q_flat(h) | turn(q_turn(h))] . [c | k_turn]) * scale
// so attention runs with one key/value head of size R + r whose cached row is [c | k_turn]; the query of head h
// is [W_uk(h)^T q_flat(h) | turn(q_turn(h))] (the first part is a product of its own), and the value is c:
// the first R numbers of what attention returns, which W_uv(h) then turns into the head's output.
//
// latent_prepare, one CTA per token: unit-RMS norm and gain of c in float32, the turn of the shared key part,
// both into the token's place in the pages; the turning parts of the queries into their place in the attention
// queries.  Pairs are neighbours (2i, 2i + 1), i < rot_dims / 2, angle p * inv_freq[i]; the other r - rot_dims
// numbers pass.
//
// sigmoid_gate: heads[t, j] *= 1 / (1 + exp(-g[t, j / span])) in float32 (span 1: a gate per number; span = a head's
// size: one gate per head).
#include "common.cuh"

namespace ps {

constexpr int LATENT_MAX_PAIRS = 256;

template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ down, int down_stride,
                      const float* __restrict__ gain, float eps, const float2* __restrict__ inv_freq, int rot_dims,
                      const int* __restrict__ token_row, const int* __restrict__ positions,
                      const int* __restrict__ block_table, int bt_stride, T* __restrict__ pool, long long page_stride,
                      int page_size, T* __restrict__ q_out, int q_out_stride, int n_heads, int flat, int turning,
                      int rank) {
    pdl_prologue();
    q = pdl_fresh(q);
    down = pdl_fresh(down);
    __shared__ float2 turn[LATENT_MAX_PAIRS];
    __shared__ float red[8];
    __shared__ float inv_shared;
    const int t = blockIdx.x;
    const int p = positions[t];
    const int half = rot_dims >> 1;
    const float pos = (float)p;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        // the angle p * f to more than one float: f comes as (high, low) parts, the product's rounding error is
        // recovered with an fma, and what does not fit the float that sincosf takes is applied to first order
        // (at position 1,000 a rounded angle is off by up to 3e-5 radians, which the scores would show)
        const float2 f = inv_freq[i];
        const float high = pos * f.x;
        const float low = fmaf(pos, f.x, -high) + pos * f.y;
        float sn, cs;
        sincosf(high, &sn, &cs);
        turn[i] = make_float2(fmaf(-low, sn, cs), fmaf(low, cs, sn));
    }
    const T* row = down + (size_t)t * down_stride;
    float sq = 0.f;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) {
        const float v = to_float(row[j]);
        sq += v * v;
    }
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
        inv_shared = 1.0f / sqrtf(s / (float)rank + eps);
    }
    __syncthreads();
    const float inv = inv_shared;
    const int width = rank + turning;                    // the cached row
    long long base = -1;
    if (pool) {
        const int page = block_table[(size_t)token_row[t] * bt_stride + p / page_size];
        if (page >= 0) base = (long long)page * page_stride + (long long)(p % page_size) * width;
    }
    if (base >= 0) {
        for (int j = threadIdx.x; j < rank; j += blockDim.x)
            pool[base + j] = from_float<T>(to_float(row[j]) * inv * gain[j]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float a = to_float(row[rank + 2 * i]), b = to_float(row[rank + 2 * i + 1]);
            pool[base + rank + 2 * i] = from_float<T>(a * turn[i].x - b * turn[i].y);
            pool[base + rank + 2 * i + 1] = from_float<T>(b * turn[i].x + a * turn[i].y);
        }
        for (int j = rot_dims + threadIdx.x; j < turning; j += blockDim.x) pool[base + rank + j] = row[rank + j];
    }
    // the queries' turning parts: head h reads q[h * (flat + turning) + flat ..], writes q_out[h * width + rank ..]
    const T* q_row = q + (size_t)t * q_stride;
    T* o_row = q_out + (size_t)t * q_out_stride;
    const int units = half + (turning - rot_dims);
    for (int idx = threadIdx.x; idx < n_heads * units; idx += blockDim.x) {
        const int h = idx / units, unit = idx - h * units;
        const T* src = q_row + (size_t)h * (flat + turning) + flat;
        T* dst = o_row + (size_t)h * width + rank;
        if (unit < half) {
            const float a = to_float(src[2 * unit]), b = to_float(src[2 * unit + 1]);
            dst[2 * unit] = from_float<T>(a * turn[unit].x - b * turn[unit].y);
            dst[2 * unit + 1] = from_float<T>(b * turn[unit].x + a * turn[unit].y);
        } else {
            const int j = rot_dims + (unit - half);
            dst[j] = src[j];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ heads, int heads_stride, const T* __restrict__ g, int g_stride, int rows,
                    int width, int span) {
    pdl_prologue();
    heads = pdl_fresh(heads);
    g = pdl_fresh(g);
    const long long total = (long long)rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / width), c = (int)(i - (long long)r * width);
        T* at = heads + (size_t)r * heads_stride + c;
        const float z = to_float(g[(size_t)r * g_stride + c / span]);
        *at = from_float<T>(to_float(*at) / (1.0f + expf(-z)));
    }
}

// The same by pieces of 16 bytes (8 bfloat16 or 4 float32 numbers) where every row of `heads` starts on such a
// boundary and a piece never straddles two gates (span a multiple of the piece) or reads a piece of gates (span 1).
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_pieces_kernel(T* __restrict__ heads, int heads_stride, const T* __restrict__ g, int g_stride, int rows,
                           int width, int span) {
    constexpr int V = 16 / (int)sizeof(T);
    pdl_prologue();
    heads = pdl_fresh(heads);
    g = pdl_fresh(g);
    const int pieces = width / V;
    const long long total = (long long)rows * pieces;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / pieces), c = (int)(i - (long long)r * pieces) * V;
        T* at = heads + (size_t)r * heads_stride + c;
        uint4 packed = *reinterpret_cast<const uint4*>(at);
        T* v = reinterpret_cast<T*>(&packed);
        if (span == 1) {
            const uint4 gates = *reinterpret_cast<const uint4*>(g + (size_t)r * g_stride + c);
            const T* z = reinterpret_cast<const T*>(&gates);
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = from_float<T>(to_float(v[j]) / (1.0f + expf(-to_float(z[j]))));
        } else {
            const float below = 1.0f + expf(-to_float(g[(size_t)r * g_stride + c / span]));
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = from_float<T>(to_float(v[j]) / below);
        }
        *reinterpret_cast<uint4*>(at) = packed;
    }
}

}  // namespace ps

// q [T, n_heads * (flat + turning)], down [T, rank + turning] (row views of the projection's output);
// gain float32 [rank]; inv_freq float32 [rot_dims / 2][2]: every frequency as a float and the float nearest to
// what the first one misses; pool: the layer's single cache plane
// [pages, 1, page_size, rank + turning] with page_stride elements between pages (null: no cache write);
// q_out [T, n_heads * (rank + turning)]: only the last `turning` numbers of every head are written.
PS_EXPORT int ps_latent_prepare(const void* q, int q_stride, const void* down, int down_stride, const float* gain,
                                float eps, const float* inv_freq, int rot_dims, const int* token_row,
                                const int* positions, const int* block_table, int bt_stride, void* pool,
                                long long page_stride, int page_size, void* q_out, int q_out_stride, int T,
                                int n_heads, int flat, int turning, int rank, int dtype, void* stream) {
    if (T <= 0) return PS_OK;
    if (n_heads <= 0 || flat < 0 || turning < 0 || rank <= 0 || rot_dims < 0 || rot_dims > turning || (rot_dims & 1))
        return PS_ERR_BAD_ARGUMENT;
    if (!q || !down || !gain || !positions || !q_out || (rot_dims > 0 && !inv_freq)) return PS_ERR_BAD_ARGUMENT;
    if (pool && (!token_row || !block_table || page_size <= 0)) return PS_ERR_BAD_ARGUMENT;
    if (rot_dims / 2 > ps::LATENT_MAX_PAIRS || ((uintptr_t)inv_freq & 7)) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = rank + n_heads * turning >= 256 ? 256 : 128;
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::latent_prepare_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)q, q_stride,
                              (const float*)down, down_stride, gain, eps, (const float2*)inv_freq, rot_dims, token_row,
                              positions, block_table, bt_stride, (float*)pool, page_stride, page_size, (float*)q_out,
                              q_out_stride, n_heads, flat, turning, rank);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::latent_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s,
                              (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)down, down_stride, gain, eps,
                              (const float2*)inv_freq, rot_dims, token_row, positions, block_table, bt_stride, (__nv_bfloat16*)pool,
                              page_stride, page_size, (__nv_bfloat16*)q_out, q_out_stride, n_heads, flat, turning,
                              rank);
    return PS_ERR_UNSUPPORTED;
}

// heads [rows, width] (in place), g [rows, width / span]: row views of the compute type.
PS_EXPORT int ps_sigmoid_gate(void* heads, int heads_stride, const void* g, int g_stride, int rows, int width,
                              int span, int dtype, void* stream) {
    if (rows <= 0 || width <= 0) return PS_OK;
    if (!heads || !g || span <= 0) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int piece = dtype == PS_F32 ? 4 : 8;
    const bool by_pieces = width % piece == 0 && heads_stride % piece == 0 && ((uintptr_t)heads & 15) == 0 &&
                           (span == 1 ? (g_stride % piece == 0 && ((uintptr_t)g & 15) == 0) : span % piece == 0);
    if (by_pieces) {
        const long long count = (long long)rows * (width / piece);
        const long long wanted = (count + 255) / 256;
        const dim3 few((unsigned)(wanted < 2368 ? wanted : 2368));
        if (dtype == PS_F32)
            return ps::launch_pdl(ps::sigmoid_gate_pieces_kernel<float>, few, dim3(256), 0, s, (float*)heads,
                                  heads_stride, (const float*)g, g_stride, rows, width, span);
        if (dtype == PS_BF16)
            return ps::launch_pdl(ps::sigmoid_gate_pieces_kernel<__nv_bfloat16>, few, dim3(256), 0, s,
                                  (__nv_bfloat16*)heads, heads_stride, (const __nv_bfloat16*)g, g_stride, rows, width,
                                  span);
        return PS_ERR_UNSUPPORTED;
    }
    const long long total = (long long)rows * width;
    const long long blocks = (total + 255) / 256;
    const dim3 grid((unsigned)(blocks < 2368 ? blocks : 2368));
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::sigmoid_gate_kernel<float>, grid, dim3(256), 0, s, (float*)heads, heads_stride,
                              (const float*)g, g_stride, rows, width, span);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)heads,
                              heads_stride, (const __nv_bfloat16*)g, g_stride, rows, width, span);
    return PS_ERR_UNSUPPORTED;
}
