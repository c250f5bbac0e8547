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
