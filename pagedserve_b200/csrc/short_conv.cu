// A short causal convolution over time on every channel of a projection, with the tail of each sequence kept as state.
//
//     y_t[c] = sum_{j < taps} w[c][j] * u_(t - taps + 1 + j)[c],      u = 0 before the sequence's first token
//
// u is the projection's float32 output for the step's tokens; what lies before an entry's first token of this step
// comes from the request's slot, which holds its last taps - 1 projected rows (oldest first; zeros when the request
// is admitted).  Channels from `conv_channels` on have no convolution and are passed through (a gate's columns that
// ride in the same product).  The result is written in the compute type.
//
// Blending of values (optional), on the channels [mix_lo, mix_lo + mix_heads * head_slot): they are heads of
// `head_slot` numbers of which the first `head_values` count.  mode 1: the convolved values are also stored, float32,
// in `shared_values` [T, mix_heads * head_values]; mode 2: y <- (1 - m) y + m * shared_values[t], m = *mix.
//
// short_conv_keep, after it: the slot receives the last taps - 1 projected rows of the sequence (rows of this step,
// and older kept rows moved up where the entry brought fewer than taps - 1 tokens).  Two launches, because every
// token of an entry may still read the old rows.
#include "common.cuh"

namespace ps {

constexpr int SHORT_CONV_MAX_TAPS = 16;

template <typename TC>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float* __restrict__ u, long long u_stride, const float* __restrict__ weight, int taps,
                  int conv_channels, int channels, const float* __restrict__ kept, long long kept_stride,
                  const int* __restrict__ token_item, const int* __restrict__ q_start, const int* __restrict__ item_slot,
                  TC* __restrict__ out, long long out_stride, int mode, int mix_lo, int mix_heads, int head_slot,
                  int head_values, float* __restrict__ shared_values, const float* __restrict__ mix, int tokens) {
    pdl_prologue();
    u = pdl_fresh(u);
    shared_values = pdl_fresh(shared_values);
    const long long total = (long long)tokens * channels;
    const float blend = mode == 2 ? *mix : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / channels), c = (int)(i - (long long)t * channels);
        float y;
        if (c >= conv_channels) {
            y = u[(size_t)t * u_stride + c];
        } else {
            const int item = token_item[t];
            const int first = q_start[item];
            const float* old = kept + (size_t)item_slot[item] * kept_stride;
            y = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int source = t - (taps - 1) + j;
                // kept row k holds the projection of the token (taps - 1 - k) places before the entry's first
                const float v = source >= first ? u[(size_t)source * u_stride + c]
                                                : old[(size_t)(taps - 1 - (first - source)) * conv_channels + c];
                y = fmaf(weight[(size_t)c * taps + j], v, y);
            }
            if (mode) {
                const int local = c - mix_lo;
                if (local >= 0 && local < mix_heads * head_slot) {
                    const int head = local / head_slot, place = local - head * head_slot;
                    if (place < head_values) {
                        float* common = shared_values + (size_t)t * mix_heads * head_values + head * head_values + place;
                        if (mode == 1) *common = y;
                        else y = (1.0f - blend) * y + blend * *common;
                    }
                }
            }
        }
        out[(size_t)t * out_stride + c] = from_float<TC>(y);
    }
}

// The same for widths, strides and addresses that are multiples of four numbers and a convolution of TAPS taps known
// when the kernel is built: a thread owns four neighbouring channels and walks a run of consecutive tokens, holding the
// last TAPS - 1 projected rows of its channels in registers, so every number of u is fetched once (and TAPS - 1
// rows again where a run begins); the taps of its channels stay in registers for the whole run.  Where a run meets an
// entry's first token the held rows are replaced by the request's kept rows.
template <typename TC> __device__ __forceinline__ void store4(TC* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = packed;
}

constexpr int SHORT_CONV_THREADS = 128;

template <typename TC, int TAPS>
__global__ void __launch_bounds__(SHORT_CONV_THREADS)
short_conv_runs_kernel(const float* __restrict__ u, long long u_stride, const float* __restrict__ weight,
                       int conv_channels, int channels, const float* __restrict__ kept, long long kept_stride,
                       const int* __restrict__ token_item, const int* __restrict__ q_start,
                       const int* __restrict__ item_slot, TC* __restrict__ out, long long out_stride, int mode, int mix_lo,
                       int mix_heads, int head_slot, int head_values, float* __restrict__ shared_values,
                       const float* __restrict__ mix, int tokens, int run) {
    const int c = 4 * (blockIdx.x * SHORT_CONV_THREADS + threadIdx.x);
    const int t0 = blockIdx.y * run, t1 = min(t0 + run, tokens);
    const bool convolved = c < conv_channels;
    // the taps of the thread's four channels: static for the step, fetched before the wait
    float w[4][TAPS];
    if (convolved && c < channels) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < TAPS; ++j) w[i][j] = weight[(size_t)(c + i) * TAPS + j];
    }
    const float blend = mode == 2 ? *mix : 0.f;
    pdl_prologue();
    u = pdl_fresh(u);
    shared_values = pdl_fresh(shared_values);
    if (c >= channels) return;
    if (!convolved) {
        for (int t = t0; t < t1; ++t) {
            const float4 v = *reinterpret_cast<const float4*>(u + (size_t)t * u_stride + c);
            const float y[4] = {v.x, v.y, v.z, v.w};
            store4<TC>(out + (size_t)t * out_stride + c, y);
        }
        return;
    }
    // where the values that are blended lie among the thread's channels (whole quads: the launcher sees to that)
    int common = -1;
    if (mode) {
        const int local = c - mix_lo;
        if (local >= 0 && local < mix_heads * head_slot) {
            const int head = local / head_slot, place = local - head * head_slot;
            if (place < head_values) common = head * head_values + place;
        }
    }
    float4 held[TAPS > 1 ? TAPS - 1 : 1];                         // held[k]: the row k + 1 tokens back
    int first = -1;
    for (int t = t0; t < t1; ++t) {
        const int item = token_item[t];
        const int start = q_start[item];
        if (t == t0 || t == start) {
            const float* old = kept + (size_t)item_slot[item] * kept_stride;
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) {
                const int source = t - 1 - k;
                held[k] = source >= start ? *reinterpret_cast<const float4*>(u + (size_t)source * u_stride + c)
                                          : *reinterpret_cast<const float4*>(old + (size_t)(TAPS - 1 - (start - source)) * conv_channels + c);
            }
            first = start;
        }
        const float4 now = *reinterpret_cast<const float4*>(u + (size_t)t * u_stride + c);
        float y[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j) {                      // tap j reads the row TAPS - 1 - j tokens back
            const float4 v = held[TAPS - 2 - j];
            y[0] = fmaf(w[0][j], v.x, y[0]); y[1] = fmaf(w[1][j], v.y, y[1]);
            y[2] = fmaf(w[2][j], v.z, y[2]); y[3] = fmaf(w[3][j], v.w, y[3]);
        }
        y[0] = fmaf(w[0][TAPS - 1], now.x, y[0]); y[1] = fmaf(w[1][TAPS - 1], now.y, y[1]);
        y[2] = fmaf(w[2][TAPS - 1], now.z, y[2]); y[3] = fmaf(w[3][TAPS - 1], now.w, y[3]);
#pragma unroll
        for (int k = TAPS - 2; k > 0; --k) held[k] = held[k - 1];
        if (TAPS > 1) held[0] = now;
        if (common >= 0) {
            float* place = shared_values + (size_t)t * mix_heads * head_values + common;
            if (mode == 1) {
                *reinterpret_cast<float4*>(place) = make_float4(y[0], y[1], y[2], y[3]);
            } else {
                const float4 other = *reinterpret_cast<const float4*>(place);
                y[0] = (1.0f - blend) * y[0] + blend * other.x; y[1] = (1.0f - blend) * y[1] + blend * other.y;
                y[2] = (1.0f - blend) * y[2] + blend * other.z; y[3] = (1.0f - blend) * y[3] + blend * other.w;
            }
        }
        store4<TC>(out + (size_t)t * out_stride + c, y);
    }
    (void)first;
}

__global__ void __launch_bounds__(256)
short_conv_keep_kernel(const float* __restrict__ u, long long u_stride, int taps, int conv_channels,
                       float* __restrict__ kept, long long kept_stride, const int* __restrict__ q_start,
                       const int* __restrict__ item_slot) {
    const int item = blockIdx.y;
    const int first = q_start[item], count = q_start[item + 1] - first;
    pdl_prologue();
    u = pdl_fresh(u);
    if (count <= 0) return;
    float* rows = kept + (size_t)item_slot[item] * kept_stride;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < conv_channels; c += gridDim.x * blockDim.x) {
        // new row k is the token at place count - (taps - 1) + k of the entry; before the entry's first token that
        // is the old row k + count, which lies above every row written so far
        for (int k = 0; k < taps - 1; ++k) {
            const int place = count - (taps - 1) + k;
            rows[(size_t)k * conv_channels + c] = place >= 0 ? u[(size_t)(first + place) * u_stride + c]
                                                             : rows[(size_t)(k + count) * conv_channels + c];
        }
    }
}

}  // namespace ps

// u float32 [T, channels] rows (u_stride apart); weight float32 [conv_channels, taps]; kept float32
// [slots, (taps - 1) * conv_channels] rows (kept_stride apart; may be null when taps = 1); out [T, channels] rows of
// `dtype`.  mode 0: no blending; 1: store the convolved values; 2: blend with the stored ones by *mix.
PS_EXPORT int ps_short_conv(const float* u, long long u_stride, const float* weight, int taps, int conv_channels,
                            int channels, const float* kept, long long kept_stride, const int* token_item,
                            const int* q_start, const int* item_slot, void* out, long long out_stride, int mode,
                            int mix_lo, int mix_heads, int head_slot, int head_values, float* shared_values,
                            const float* mix, int T, int dtype, void* stream) {
    if (T <= 0 || channels <= 0) return PS_OK;
    if (!u || !out || conv_channels < 0 || conv_channels > channels || taps < 1) return PS_ERR_BAD_ARGUMENT;
    if (conv_channels && (!weight || !token_item || !q_start || !item_slot || (taps > 1 && !kept)))
        return PS_ERR_BAD_ARGUMENT;
    if (mode < 0 || mode > 2 || (mode && (!shared_values || head_slot <= 0 || head_values <= 0 || head_values > head_slot)))
        return PS_ERR_BAD_ARGUMENT;
    if (mode == 2 && !mix) return PS_ERR_BAD_ARGUMENT;
    if (taps > ps::SHORT_CONV_MAX_TAPS) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    // quads of channels over runs of tokens, where every boundary between kinds of channels falls between quads
    const int elem = dtype == PS_F32 ? 4 : 2;
    const bool quads = taps <= 4 && conv_channels > 0 && channels % 4 == 0 && conv_channels % 4 == 0 && u_stride % 4 == 0 &&
                       out_stride % 4 == 0 && kept_stride % 4 == 0 && !((uintptr_t)u & 15) && !((uintptr_t)kept & 15) &&
                       !((uintptr_t)out & (uintptr_t)(4 * elem - 1)) &&
                       (!mode || (mix_lo % 4 == 0 && head_slot % 4 == 0 && head_values % 4 == 0 &&
                                  !((uintptr_t)shared_values & 15)));
    if (quads && (dtype == PS_F32 || dtype == PS_BF16)) {
        // runs of 16 tokens re-read (taps - 1) / 16 of the rows; shorter runs where the step has few tokens
        const int columns = (channels / 4 + ps::SHORT_CONV_THREADS - 1) / ps::SHORT_CONV_THREADS;
        int run = 16;
        while (run > 1 && (long long)columns * ((T + run - 1) / run) < 296) run >>= 1;
        const dim3 grid(columns, (T + run - 1) / run), block(ps::SHORT_CONV_THREADS);
#define PS_CONV_RUNS(TYPE, TAPS)                                                                                      \
    return ps::launch_pdl(ps::short_conv_runs_kernel<TYPE, TAPS>, grid, block, 0, s, u, u_stride, weight, conv_channels, \
                          channels, kept, kept_stride, token_item, q_start, item_slot, (TYPE*)out, out_stride, mode,     \
                          mix_lo, mix_heads, head_slot, head_values, shared_values, mix, T, run)
#define PS_CONV_TAPS(TYPE)                                                                                            \
    switch (taps) {                                                                                                   \
        case 1: PS_CONV_RUNS(TYPE, 1);                                                                                \
        case 2: PS_CONV_RUNS(TYPE, 2);                                                                                \
        case 3: PS_CONV_RUNS(TYPE, 3);                                                                                \
        default: PS_CONV_RUNS(TYPE, 4);                                                                               \
    }
        if (dtype == PS_F32) PS_CONV_TAPS(float)
        PS_CONV_TAPS(__nv_bfloat16)
#undef PS_CONV_TAPS
#undef PS_CONV_RUNS
    }
    const long long total = (long long)T * channels;
    const long long blocks = (total + 255) / 256;
    const dim3 grid((unsigned)(blocks < 4736 ? blocks : 4736));
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::short_conv_kernel<float>, grid, dim3(256), 0, s, u, u_stride, weight, taps,
                              conv_channels, channels, kept, kept_stride, token_item, q_start, item_slot, (float*)out,
                              out_stride, mode, mix_lo, mix_heads, head_slot, head_values, shared_values, mix, T);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::short_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, u, u_stride, weight, taps,
                              conv_channels, channels, kept, kept_stride, token_item, q_start, item_slot,
                              (__nv_bfloat16*)out, out_stride, mode, mix_lo, mix_heads, head_slot, head_values,
                              shared_values, mix, T);
    return PS_ERR_UNSUPPORTED;
}

PS_EXPORT int ps_short_conv_keep(const float* u, long long u_stride, int taps, int conv_channels, float* kept,
                                 long long kept_stride, const int* q_start, const int* item_slot, int items,
                                 void* stream) {
    if (items <= 0 || taps <= 1 || conv_channels <= 0) return PS_OK;
    if (!u || !kept || !q_start || !item_slot) return PS_ERR_BAD_ARGUMENT;
    if (taps > ps::SHORT_CONV_MAX_TAPS) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    int blocks = (conv_channels + 255) / 256;
    if (blocks > 64) blocks = 64;
    return ps::launch_pdl(ps::short_conv_keep_kernel, dim3(blocks, items), dim3(256), 0, s, u, u_stride, taps,
                          conv_channels, kept, kept_stride, q_start, item_slot);
}
