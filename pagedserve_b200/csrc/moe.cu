// Routed experts: the router and the gated inner activation.
//
// moe_route, one CTA per token, float32 throughout:
//     z = W_router h                    (E numbers; the operands may be bfloat16, sums are float32)
//     s = softmax(z) over all E experts, or s = sigmoid(z) expert by expert (score_kind 1)
//     with groups: the experts are `groups` runs of E / groups neighbours; a group's mark is its largest s; only
//     experts of the `keep` groups with the largest marks stand for election
//     the `top` largest s among them are chosen (ties: the lower index), and their weights are s / (sum of the
//     chosen s + 1e-20), or the chosen s themselves (normalize 0); the lanes of one warp hold the scores and run
//     every round together
//     shared gate: sigmoid(w_sg . h), one number per token (where the layer has a shared expert)
// Results: dense weights [T, E] (0 where an expert is not chosen), the chosen experts and their weights
// [T, top], and the shared gate [T].
//
// The inner activation of a gated expert from its gate and up pre-activations g, u and the token's weight w
// (GateForm):
//     kind 0:  silu(g) * u * w                                   (the weight scales the expert's output)
//     kind 1:  g' = min(w g, limit), u' = clamp(w u, -limit, limit);  g' * sigmoid(alpha g') * (u' + 1)
//              (the weight scales the expert's input: without biases W (w h) = w (W h), so it is applied to the
//              pre-activations in float32; the shared expert's columns have a limit of their own)
// moe_gate_mul: inner[t, c] = silu(gate) * up * weight[t, expert of column c] over one stacked product of all
// experts: expert e's block of 2 F columns is its gate columns, then its up columns; the shared expert's block
// follows the experts' (weight = the shared gate, or 1 without one; E = 0: a dense gated feed-forward).  inner's columns [e * F, (e + 1) * F) belong to expert e, those
// from E * F on to the shared expert.  Products in float32, rounded once.
//
// With many tokens the rows are sorted by expert instead (moe_plan, moe_gather, the products over tiles that
// choose their expert's matrix, moe_gate_mul_rows, moe_combine): every token passes only through its own experts.
#include "common.cuh"

namespace ps {

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_WARPS = 4;
constexpr int MOE_BATCH = 16;                     // experts whose sums a lane keeps in registers at a time

// eight neighbouring elements as floats: one 16-byte access of bfloat16, two of float32
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

struct GateForm {
    int kind;                 // 0: silu(g) u w; 1: clamped, weight on the input (see the top of the file)
    float limit;              // kind 1: the routed experts' limit
    float shared_limit;       // kind 1: the shared expert's
    float alpha;              // kind 1: the sigmoid's slope
};

__device__ __forceinline__ float gated_inner(float g, float u, float w, int kind, float limit, float alpha) {
    if (kind == 0) return silu(g) * u * w;
    g = fminf(g * w, limit);
    u = fminf(fmaxf(u * w, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32, 8)
moe_route_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ router, int router_stride,
                 const T* __restrict__ shared_gate_w, float* __restrict__ dense, int* __restrict__ chosen,
                 float* __restrict__ chosen_w, float* __restrict__ shared_gate, int tokens, int W, int E, int top,
                 int groups, int keep, int by8, const float* __restrict__ raw, int raw_stride,
                 const float* __restrict__ gain, float eps, T* __restrict__ x_out, int score_kind, int normalize,
                 const float* __restrict__ correction) {
    pdl_prologue();
    x = pdl_fresh(x);
    raw = pdl_fresh(raw);
    // One CTA per token.  The E logits (and the shared gate's, as one more row) are dot products over the row: the
    // threads of the CTA share the row's columns, so that with eight numbers per thread a row of 1,024 is one round
    // of loads, all in flight together; partial sums meet in shared memory; warp 0 then holds the election.
    __shared__ float score[MOE_MAX_EXPERTS + 1];
    __shared__ float partial[MOE_WARPS][MOE_BATCH];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    if (raw) {
        // The RMS norm in front, folded in: this CTA norms its token's float32 row (x / sqrt(mean(x^2) + eps) * gain),
        // leaves the rounded row in x_out for the experts' products, and reads its own numbers back below (every
        // thread the columns it wrote itself).
        __shared__ float square[MOE_WARPS];
        __shared__ float inv_shared;
        const float* source = raw + (size_t)t * raw_stride;
        T* target = x_out + (size_t)t * x_stride;
        float sq = 0.f;
        if (by8) {
            for (int j = 8 * threadIdx.x; j < W; j += 8 * MOE_WARPS * 32) {
                float v[8];
                load8(source + j, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) sq = fmaf(v[i], v[i], sq);
            }
        } else {
            for (int j = threadIdx.x; j < W; j += MOE_WARPS * 32) sq = fmaf(source[j], source[j], sq);
        }
        sq = warp_sum(sq);
        if (lane == 0) square[warp] = sq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.f;
            for (int w = 0; w < MOE_WARPS; ++w) total += square[w];
            inv_shared = 1.0f / sqrtf(total / (float)W + eps);
        }
        __syncthreads();
        const float inv = inv_shared;
        if (by8) {
            for (int j = 8 * threadIdx.x; j < W; j += 8 * MOE_WARPS * 32) {
                float v[8], g[8];
                load8(source + j, v);
                load8(gain + j, g);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * g[i];
                store8(target + j, v);
            }
        } else {
            for (int j = threadIdx.x; j < W; j += MOE_WARPS * 32) target[j] = from_float<T>(source[j] * inv * gain[j]);
        }
        __syncthreads();
        x = pdl_fresh(static_cast<const T*>(x_out));      // (a pointer the compiler cannot tie to the stores above)
    }
    const T* row = x + (size_t)t * x_stride;
    const int rows = E + (shared_gate_w ? 1 : 0);
    for (int e0 = 0; e0 < rows; e0 += MOE_BATCH) {
        float acc[MOE_BATCH];
#pragma unroll
        for (int b = 0; b < MOE_BATCH; ++b) acc[b] = 0.f;
        if (by8) {
            for (int j = 8 * threadIdx.x; j < W; j += 8 * MOE_WARPS * 32) {
                float xv[8];
                load8(row + j, xv);
#pragma unroll
                for (int b = 0; b < MOE_BATCH; ++b) {
                    if (e0 + b < rows) {
                        const T* w = e0 + b < E ? router + (size_t)(e0 + b) * router_stride : shared_gate_w;
                        float wv[8];
                        load8(w + j, wv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[b] = fmaf(xv[i], wv[i], acc[b]);
                    }
                }
            }
        } else {
            for (int j = threadIdx.x; j < W; j += MOE_WARPS * 32) {
                const float xv = to_float(row[j]);
#pragma unroll
                for (int b = 0; b < MOE_BATCH; ++b) {
                    if (e0 + b < rows) {
                        const T* w = e0 + b < E ? router + (size_t)(e0 + b) * router_stride : shared_gate_w;
                        acc[b] = fmaf(xv, to_float(w[j]), acc[b]);
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < MOE_BATCH; ++b) {
            const float total = warp_sum(acc[b]);
            if (lane == 0) partial[warp][b] = total;
        }
        __syncthreads();
        if (threadIdx.x < MOE_BATCH && e0 + threadIdx.x < rows) {
            float total = 0.f;
#pragma unroll
            for (int w = 0; w < MOE_WARPS; ++w) total += partial[w][threadIdx.x];
            score[e0 + threadIdx.x] = total;
        }
        __syncthreads();
    }
    if (warp != 0) return;
    if (shared_gate_w && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-score[E]));
    // ---- the election, by the lanes of warp 0 together: lane l holds the experts l, l + 32, ...
    constexpr int PER_LANE = MOE_MAX_EXPERTS / 32;
    float mine[PER_LANE];
    float top_z = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int e = lane + 32 * i;
        mine[i] = e < E ? score[e] : -INFINITY;
        top_z = fmaxf(top_z, mine[i]);
    }
    top_z = warp_max(top_z);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        if (score_kind == 1) mine[i] = lane + 32 * i < E ? 1.0f / (1.0f + expf(-mine[i])) : 0.f;      // sigmoid
        else mine[i] = lane + 32 * i < E ? expf(mine[i] - top_z) : 0.f;
        sum += mine[i];
    }
    sum = warp_sum(sum);
    const float inv = score_kind == 1 ? 1.0f : 1.0f / sum;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int e = lane + 32 * i;
        mine[i] = e < E ? mine[i] * inv : -INFINITY;           // the scores; -inf: no such expert
        if (e < E) {
            score[e] = mine[i];
            dense[(size_t)t * E + e] = 0.f;
            // a correction moves the election only: an expert stands with score + correction, its weight stays the score
            if (correction) mine[i] += correction[e];
        }
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        // a group's mark is its largest score; groups - keep times the open group with the lowest mark is closed
        // (ties: the higher index goes, so that the lower index stays, as in the election below)
        const int per = E / groups;
        __shared__ float group_mark[MOE_MAX_EXPERTS];
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY;
            for (int j = 0; j < per; ++j) m = fmaxf(m, score[g * per + j]);
            group_mark[g] = m;
        }
        __syncwarp();
        for (int drop = 0; drop < groups - keep; ++drop) {
            float worst = INFINITY;
            int worst_g = -1;
            for (int g = lane; g < groups; g += 32) {
                const float m = group_mark[g];
                if (m <= worst && m != INFINITY) { worst = m; worst_g = g; }      // later (higher) g wins ties
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float other = __shfl_xor_sync(0xffffffffu, worst, o);
                const int other_g = __shfl_xor_sync(0xffffffffu, worst_g, o);
                if (other_g >= 0 && (worst_g < 0 || other < worst || (other == worst && other_g > worst_g))) {
                    worst = other;
                    worst_g = other_g;
                }
            }
            if (worst_g < 0) break;
            if (lane == 0) group_mark[worst_g] = INFINITY;       // closed
            __syncwarp();
        }
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < E && group_mark[e / per] == INFINITY) mine[i] = -INFINITY;
        }
    }
    __shared__ int winner[MOE_MAX_EXPERTS];
    __shared__ float winner_score[MOE_MAX_EXPERTS];
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = -1;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i)
            if (mine[i] > best) { best = mine[i]; best_e = lane + 32 * i; }       // rising e: the lower index wins ties
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, o);
            const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (other_e >= 0 && (best_e < 0 || other > best || (other == best && other_e < best_e))) {
                best = other;
                best_e = other_e;
            }
        }
        // every lane now knows the winner; its owner takes it out of the running
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i)
            if (best_e == lane + 32 * i) mine[i] = -INFINITY;
        if (lane == 0) {
            winner[k] = best_e;                                  // -1: fewer open experts than `top`
            winner_score[k] = best_e >= 0 ? (correction ? score[best_e] : best) : 0.f;
        }
        if (best_e >= 0) total += correction ? score[best_e] : best;
    }
    __syncwarp();
    const float scale = normalize ? 1.0f / (total + 1e-20f) : 1.0f;
    for (int k = lane; k < top; k += 32) {
        const int e = winner[k];
        const float w = winner_score[k] * scale;
        chosen[(size_t)t * top + k] = e;
        chosen_w[(size_t)t * top + k] = w;
        if (e >= 0) dense[(size_t)t * E + e] = w;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_mul_kernel(const T* __restrict__ gate_up, int gu_stride, const float* __restrict__ dense,
                    const float* __restrict__ shared_gate, T* __restrict__ inner, int inner_stride, int tokens,
                    int columns, int E, int F, int by8, GateForm form) {
    pdl_prologue();
    gate_up = pdl_fresh(gate_up);
    dense = pdl_fresh(dense);
    shared_gate = pdl_fresh(shared_gate);
    const long long total = (long long)tokens * columns;
    const int shared_ff = columns - E * F;
    if (by8) {                                  // eight neighbouring columns (of one expert) per thread and turn
        const int groups = columns >> 3;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)tokens * groups;
             i += (long long)gridDim.x * blockDim.x) {
            const int t = (int)(i / groups), c = (int)(i - (long long)t * groups) << 3;
            const int e = c < E * F ? c / F : E;
            const float w = e < E ? dense[(size_t)t * E + e] : (shared_gate ? shared_gate[t] : 1.0f);
            const float limit = e < E ? form.limit : form.shared_limit;
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (w != 0.f) {
                const int j = c - e * F;
                const T* block = gate_up + (size_t)t * gu_stride + 2 * (size_t)e * F;
                float g[8], u[8];
                load8(block + j, g);
                load8(block + (e < E ? F : shared_ff) + j, u);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = gated_inner(g[k], u[k], w, form.kind, limit, form.alpha);
            }
            store8(inner + (size_t)t * inner_stride + c, v);
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / columns), c = (int)(i - (long long)t * columns);
        const int e = c < E * F ? c / F : E;
        const float w = e < E ? dense[(size_t)t * E + e] : (shared_gate ? shared_gate[t] : 1.0f);
        float v = 0.f;
        if (w != 0.f) {
            // an expert's block of the stacked product is its gate columns, then its up columns
            const int j = c - e * F;
            const T* block = gate_up + (size_t)t * gu_stride + 2 * (size_t)e * F;
            v = gated_inner(to_float(block[j]), to_float(block[(e < E ? F : shared_ff) + j]), w, form.kind,
                            e < E ? form.limit : form.shared_limit, form.alpha);
        }
        inner[(size_t)t * inner_stride + c] = from_float<T>(v);
    }
}

// ---- rows sorted by expert (steps of many tokens) ----
// moe_plan, one CTA: every (token, chosen expert) pair gets a row in a buffer in which the rows of one expert lie
// together and every expert's run starts on a multiple of `tile` rows (the row count of a product's tile), so that a
// tile of the product belongs to one expert.  row_of[t * top + k]: the pair's row (-1: no expert);
// row_token[row] / row_weight[row]: the token and the weight of a row (-1 / 0 for the padding between runs);
// tile_expert[tile]: the expert of a tile of rows, -1 behind the last run.  The order of an expert's rows is
// whatever the atomics give: no result depends on it, every row is computed by itself.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ chosen, const float* __restrict__ chosen_w, int pairs, int E, int tile,
                int rows_cap, int* __restrict__ row_of, int* __restrict__ row_token, float* __restrict__ row_weight,
                int* __restrict__ tile_expert, int top) {
    __shared__ int count[MOE_MAX_EXPERTS], start[MOE_MAX_EXPERTS + 1], cursor[MOE_MAX_EXPERTS];
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
    __syncthreads();
    pdl_prologue();
    chosen = pdl_fresh(chosen);
    chosen_w = pdl_fresh(chosen_w);
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            at += (count[e] + tile - 1) / tile * tile;
        }
        start[E] = at;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < rows_cap; r += blockDim.x) {
        row_token[r] = -1;
        row_weight[r] = 0.f;
    }
    for (int t = threadIdx.x; t < rows_cap / tile; t += blockDim.x) {
        const int first = t * tile;
        int expert = -1;
        for (int e = 0; e < E; ++e)
            if (first >= start[e] && first < start[e + 1] && count[e] > 0 && first < start[e] + count[e]) expert = e;
        tile_expert[t] = expert;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        int row = -1;
        if (e >= 0 && e < E) {
            row = start[e] + atomicAdd(&cursor[e], 1);
            row_token[row] = i / top;
            row_weight[row] = chosen_w[i];
        }
        row_of[i] = row;
    }
}

// rows[r] = x[row_token[r]] (zeros for the padding rows); 16 bytes per thread and turn.
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const T* __restrict__ x, int x_stride, const int* __restrict__ row_token, T* __restrict__ rows,
                  int rows_stride, int W, int by16) {
    pdl_prologue();
    x = pdl_fresh(x);
    row_token = pdl_fresh(row_token);
    const int r = blockIdx.x;
    const int t = row_token[r];
    T* dst = rows + (size_t)r * rows_stride;
    const T* src = x + (size_t)(t < 0 ? 0 : t) * x_stride;
    if (by16) {                                 // 16 bytes per thread and turn
        constexpr int PER = 16 / sizeof(T);
        const uint4 zero = make_uint4(0, 0, 0, 0);
        for (int c = threadIdx.x * PER; c < W; c += blockDim.x * PER)
            *reinterpret_cast<uint4*>(dst + c) = t < 0 ? zero : *reinterpret_cast<const uint4*>(src + c);
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = t < 0 ? from_float<T>(0.f) : src[c];
}

// inner[r, j] = silu(gate_up[r, j]) * gate_up[r, F + j] * row_weight[r], or the other form of GateForm
template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_mul_rows_kernel(const T* __restrict__ gate_up, int gu_stride, const float* __restrict__ row_weight,
                         T* __restrict__ inner, int inner_stride, int rows, int F, int by8, GateForm form) {
    pdl_prologue();
    gate_up = pdl_fresh(gate_up);
    row_weight = pdl_fresh(row_weight);
    const long long total = (long long)rows * F;
    if (by8) {
        const int groups = F >> 3;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)rows * groups;
             i += (long long)gridDim.x * blockDim.x) {
            const int r = (int)(i / groups), j = (int)(i - (long long)r * groups) << 3;
            const float w = row_weight[r];
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (w != 0.f) {
                const T* row = gate_up + (size_t)r * gu_stride;
                float g[8], u[8];
                load8(row + j, g);
                load8(row + F + j, u);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = gated_inner(g[k], u[k], w, form.kind, form.limit, form.alpha);
            }
            store8(inner + (size_t)r * inner_stride + j, v);
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / F), j = (int)(i - (long long)r * F);
        const float w = row_weight[r];
        float v = 0.f;
        if (w != 0.f) {
            const T* row = gate_up + (size_t)r * gu_stride;
            v = gated_inner(to_float(row[j]), to_float(row[F + j]), w, form.kind, form.limit, form.alpha);
        }
        inner[(size_t)r * inner_stride + j] = from_float<T>(v);
    }
}

// y[t] += sum over k (in rising order) of down[row_of[t * top + k]]
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ down, int down_stride, const int* __restrict__ row_of, int top,
                   float* __restrict__ y, int y_stride, int W, int by4) {
    pdl_prologue();
    down = pdl_fresh(down);
    row_of = pdl_fresh(row_of);
    y = pdl_fresh(y);
    const int t = blockIdx.x;
    if (by4) {
        for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
            float4 acc = *reinterpret_cast<const float4*>(y + (size_t)t * y_stride + c);
            for (int k = 0; k < top; ++k) {
                const int r = row_of[t * top + k];
                if (r < 0) continue;
                const float4 d = *reinterpret_cast<const float4*>(down + (size_t)r * down_stride + c);
                acc.x += d.x; acc.y += d.y; acc.z += d.z; acc.w += d.w;
            }
            *reinterpret_cast<float4*>(y + (size_t)t * y_stride + c) = acc;
        }
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = y[(size_t)t * y_stride + c];
        for (int k = 0; k < top; ++k) {
            const int r = row_of[t * top + k];
            if (r >= 0) acc += down[(size_t)r * down_stride + c];
        }
        y[(size_t)t * y_stride + c] = acc;
    }
}

}  // namespace ps

// x [T, W] rows of the compute type; router [E, W]; shared_gate_w [W] or null; dense float32 [T, E];
// chosen int32 [T, top]; chosen_w float32 [T, top]; shared_gate float32 [T] (written only with shared_gate_w).
// raw (may be null): float32 [T, W] rows whose RMS norm (gain float32 [W], eps) is what the router reads: the normed
// rows are then written to x (which the experts' products read) instead of being read from it.  correction (may be
// null): float32 [E] added to the scores for the election only.
PS_EXPORT int ps_moe_route(const void* x, int x_stride, const void* router, int router_stride,
                           const void* shared_gate_w, float* dense, int* chosen, float* chosen_w, float* shared_gate,
                           int T, int W, int E, int top, int groups, int keep, int dtype, const float* raw,
                           int raw_stride, const float* gain, float eps, int score_kind, int normalize,
                           const float* correction, void* stream) {
    if (T <= 0) return PS_OK;
    if (raw && !gain) return PS_ERR_BAD_ARGUMENT;
    if (W <= 0 || E <= 0 || top <= 0 || top > E || !x || !router || !dense || !chosen || !chosen_w)
        return PS_ERR_BAD_ARGUMENT;
    if (groups < 0 || (groups > 1 && (E % groups || keep <= 0 || keep > groups))) return PS_ERR_BAD_ARGUMENT;
    if (shared_gate_w && !shared_gate) return PS_ERR_BAD_ARGUMENT;
    if (score_kind < 0 || score_kind > 1) return PS_ERR_BAD_ARGUMENT;
    if (E > ps::MOE_MAX_EXPERTS) return PS_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(T), block(ps::MOE_WARPS * 32);
    // rows of the input and of the router in 32-byte units: eight numbers per access
    const int by8 = W % 8 == 0 && x_stride % 8 == 0 && router_stride % 8 == 0 && !((uintptr_t)x & 31) &&
                    !((uintptr_t)router & 31) && !((uintptr_t)shared_gate_w & 15) &&
                    (!raw || (raw_stride % 8 == 0 && !((uintptr_t)raw & 31) && !((uintptr_t)gain & 31)));
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::moe_route_kernel<float>, grid, block, 0, s, (const float*)x, x_stride,
                              (const float*)router, router_stride, (const float*)shared_gate_w, dense, chosen,
                              chosen_w, shared_gate, T, W, E, top, groups, keep, by8, raw, raw_stride, gain, eps,
                              (float*)const_cast<void*>(x), score_kind, normalize, correction);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::moe_route_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)x,
                              x_stride, (const __nv_bfloat16*)router, router_stride,
                              (const __nv_bfloat16*)shared_gate_w, dense, chosen, chosen_w, shared_gate, T, W, E, top,
                              groups, keep, by8, raw, raw_stride, gain, eps, (__nv_bfloat16*)const_cast<void*>(x),
                              score_kind, normalize, correction);
    return PS_ERR_UNSUPPORTED;
}

// gate_up [T, 2 * columns] (per expert: gates, then ups); dense float32 [T, E]; shared_gate float32 [T] (read for
// columns from E * F on); inner [T, columns].
PS_EXPORT int ps_moe_gate_mul(const void* gate_up, int gu_stride, const float* dense, const float* shared_gate,
                              void* inner, int inner_stride, int T, int columns, int E, int F, int dtype,
                              int kind, float limit, float shared_limit, float alpha, void* stream) {
    if (T <= 0 || columns <= 0) return PS_OK;
    if (!gate_up || !inner || E < 0 || (E > 0 && !dense) || F <= 0 || columns < E * F) return PS_ERR_BAD_ARGUMENT;
    if (kind < 0 || kind > 1 || (kind == 1 && !(limit > 0.f && shared_limit > 0.f))) return PS_ERR_BAD_ARGUMENT;
    const ps::GateForm form{kind, limit, shared_limit, alpha};
    cudaStream_t s = (cudaStream_t)stream;
    const int by8 = F % 8 == 0 && columns % 8 == 0 && gu_stride % 8 == 0 && inner_stride % 8 == 0 &&
                    !((uintptr_t)gate_up & 31) && !((uintptr_t)inner & 31);
    const long long total = (long long)T * (by8 ? columns / 8 : columns);
    const long long blocks = (total + 255) / 256;
    const dim3 grid((unsigned)(blocks < 4736 ? blocks : 4736));
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::moe_gate_mul_kernel<float>, grid, dim3(256), 0, s, (const float*)gate_up, gu_stride,
                              dense, shared_gate, (float*)inner, inner_stride, T, columns, E, F, by8, form);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::moe_gate_mul_kernel<__nv_bfloat16>, grid, dim3(256), 0, s,
                              (const __nv_bfloat16*)gate_up, gu_stride, dense, shared_gate, (__nv_bfloat16*)inner,
                              inner_stride, T, columns, E, F, by8, form);
    return PS_ERR_UNSUPPORTED;
}

// chosen int32 / chosen_w float32 [T * top]; row_of int32 [T * top]; row_token int32, row_weight float32 [rows_cap];
// tile_expert int32 [rows_cap / tile]; rows_cap: a multiple of tile, at least T * top + E * (tile - 1).
PS_EXPORT int ps_moe_plan(const int* chosen, const float* chosen_w, int T, int top, int E, int tile, int rows_cap,
                          int* row_of, int* row_token, float* row_weight, int* tile_expert, void* stream) {
    if (T <= 0) return PS_OK;
    if (!chosen || !chosen_w || !row_of || !row_token || !row_weight || !tile_expert || top <= 0 || E <= 0 || tile <= 0)
        return PS_ERR_BAD_ARGUMENT;
    if (E > ps::MOE_MAX_EXPERTS) return PS_ERR_UNSUPPORTED;
    if (rows_cap % tile || (long long)rows_cap < (long long)T * top + (long long)E * (tile - 1)) return PS_ERR_BAD_ARGUMENT;
    return ps::launch_pdl(ps::moe_plan_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, chosen, chosen_w, T * top,
                          E, tile, rows_cap, row_of, row_token, row_weight, tile_expert, top);
}

// x [T, W] -> rows [R, W] by row_token [R]
PS_EXPORT int ps_moe_gather(const void* x, int x_stride, const int* row_token, void* rows, int rows_stride, int R,
                            int W, int dtype, void* stream) {
    if (R <= 0 || W <= 0) return PS_OK;
    if (!x || !row_token || !rows) return PS_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int by16 = W % 8 == 0 && x_stride % 8 == 0 && rows_stride % 8 == 0 && !((uintptr_t)x & 15) &&
                     !((uintptr_t)rows & 15);
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::moe_gather_kernel<float>, dim3(R), dim3(128), 0, s, (const float*)x, x_stride,
                              row_token, (float*)rows, rows_stride, W, by16);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::moe_gather_kernel<__nv_bfloat16>, dim3(R), dim3(128), 0, s, (const __nv_bfloat16*)x,
                              x_stride, row_token, (__nv_bfloat16*)rows, rows_stride, W, by16);
    return PS_ERR_UNSUPPORTED;
}

// gate_up [R, 2 F] (gate columns, then up columns); row_weight float32 [R]; inner [R, F]
PS_EXPORT int ps_moe_gate_mul_rows(const void* gate_up, int gu_stride, const float* row_weight, void* inner,
                                   int inner_stride, int R, int F, int dtype, int kind, float limit, float alpha,
                                   void* stream) {
    if (R <= 0 || F <= 0) return PS_OK;
    if (!gate_up || !row_weight || !inner) return PS_ERR_BAD_ARGUMENT;
    if (kind < 0 || kind > 1 || (kind == 1 && !(limit > 0.f))) return PS_ERR_BAD_ARGUMENT;
    const ps::GateForm form{kind, limit, limit, alpha};
    cudaStream_t s = (cudaStream_t)stream;
    const int by8 = F % 8 == 0 && gu_stride % 8 == 0 && inner_stride % 8 == 0 && !((uintptr_t)gate_up & 31) &&
                    !((uintptr_t)inner & 31);
    const long long blocks = ((long long)R * (by8 ? F / 8 : F) + 255) / 256;
    const dim3 grid((unsigned)(blocks < 4736 ? blocks : 4736));
    if (dtype == PS_F32)
        return ps::launch_pdl(ps::moe_gate_mul_rows_kernel<float>, grid, dim3(256), 0, s, (const float*)gate_up,
                              gu_stride, row_weight, (float*)inner, inner_stride, R, F, by8, form);
    if (dtype == PS_BF16)
        return ps::launch_pdl(ps::moe_gate_mul_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, s,
                              (const __nv_bfloat16*)gate_up, gu_stride, row_weight, (__nv_bfloat16*)inner, inner_stride,
                              R, F, by8, form);
    return PS_ERR_UNSUPPORTED;
}

// down float32 [R, W]; row_of int32 [T * top]; y float32 [T, W]
PS_EXPORT int ps_moe_combine(const float* down, int down_stride, const int* row_of, int top, float* y, int y_stride,
                             int T, int W, void* stream) {
    if (T <= 0 || W <= 0) return PS_OK;
    if (!down || !row_of || !y || top <= 0) return PS_ERR_BAD_ARGUMENT;
    const int by4 = W % 4 == 0 && down_stride % 4 == 0 && y_stride % 4 == 0 && !((uintptr_t)down & 15) &&
                    !((uintptr_t)y & 15);
    return ps::launch_pdl(ps::moe_combine_kernel, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, down,
                          down_stride, row_of, top, y, y_stride, W, by4);
}
