// Routed feed-forward: a router that scores experts (sigmoid or softmax), restricts the choice to the best
// groups of neighbouring experts, and picks the `top` largest; gated experts evaluated per (token, chosen
// expert) with the expert's weights streamed once per pair; and the weighted sum of the experts' outputs.
// Router, scores and the weighted sum are 32-bit.
#include "common.cuh"

namespace lb {

// The lane-wise best (largest value, lowest index among equals) over a warp; every lane gets it.
__device__ __forceinline__ void warp_argmax(float& value, int& index) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other_value > value || (other_value == value && other_index < index)) {
            value = other_value;
            index = other_index;
        }
    }
}

// One warp per token or, with `block_per_token`, one block per token whose warps share out the experts' logits (few
// tokens: more loads on their way at once), the first warp choosing afterwards.  A logit's sum is the same either way.
//   z[e] = x . router[e] (+ bias[e])  (32-bit);   s[e] = sigmoid(z[e])   (score_kind 0),  softmax(z)[e]   (score_kind 1)  or  z[e]  (score_kind 2)
//   experts form `group_count` equal groups of neighbours; a group's score is the sum of its two largest s (of its
//   only one, in groups of one); experts outside the best `group_keep` groups cannot be chosen;
//   chosen[t, :] = the `top` eligible experts of largest s, in that order; weights[t, :] = their s (divided by their
//   sum if `renormalize` is 1; the softmax over just the chosen s if it is 2), times `weight_scale`.
//   `choice_bias` (may be null): experts (and groups) are ranked by s[e] + choice_bias[e]; the weights stay the s themselves.
//   `extra` further rows of `router` after the experts' are gates of something every token runs: extra_out[t, x] =
//   sigmoid(x_t . router[experts + x]), 32-bit like the scores.
// Shared memory per warp: s[experts], candidates[experts], group score[group_count], and the token's row in 32-bit where it is staged.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router, int* __restrict__ chosen, float* __restrict__ weights,
                                 int tokens, int width, int experts, int top, int group_count, int group_keep, int score_kind, int renormalize,
                                 float weight_scale, int row_floats, int group_floats, const float* __restrict__ bias, int block_per_token,
                                 const float* __restrict__ choice_bias, int extra, float* __restrict__ extra_out) {
    extern __shared__ __align__(16) float shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int token = block_per_token ? blockIdx.x : blockIdx.x * warps + warp;
    if (token >= tokens) return;
    const int sharers = block_per_token ? warps : 1, share = block_per_token ? warp : 0;   // the logits of experts 4 (share + i sharers) .. + 3 are this warp's
    const int logits = experts + extra;   // rows of the router
    float* scores = shared + static_cast<size_t>(block_per_token ? 0 : warp) * (experts + logits + group_floats + row_floats);   // a multiple of 4 floats per warp
    float* candidates = scores + logits;
    float* group_score = candidates + experts;   // group_floats >= group_count of them
    float* x_s = group_score + group_floats;   // row_floats = width (rounded up to a multiple of 4) if the row is staged, else 0
    const T* row = x + static_cast<size_t>(token) * width;
    if (row_floats > 0) {
        // the token's row once into shared memory (32-bit), then four experts' rows at a time, 16 bytes a lane and turn
        if (block_per_token) {
            for (int d = threadIdx.x; d < width; d += blockDim.x) x_s[d] = to_float(row[d]);
            __syncthreads();
        } else {
#pragma unroll 8
            for (int d = lane; d < width; d += 32) x_s[d] = to_float(row[d]);
            __syncwarp();
        }
        for (int e0 = 4 * share; e0 < logits; e0 += 4 * sharers) {
            float dots[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
            for (int c = 4 * lane; c < width; c += 128) {   // sixteen loads of the router's rows on their way at a time
                const float4 xv = *reinterpret_cast<const float4*>(x_s + c);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float4 w = *reinterpret_cast<const float4*>(router + static_cast<size_t>(e0 + r < logits ? e0 + r : e0) * width + c);
                    dots[r] += xv.x * w.x;
                    dots[r] += xv.y * w.y;
                    dots[r] += xv.z * w.z;
                    dots[r] += xv.w * w.w;
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float dot = warp_sum(dots[r]);
                if (lane == 0 && e0 + r < logits) scores[e0 + r] = dot;
            }
        }
    } else {
        for (int e = share; e < logits; e += sharers) {
            const float* w = router + static_cast<size_t>(e) * width;
            float dot = 0.0f;
            for (int d = lane; d < width; d += 32) dot += to_float(row[d]) * w[d];
            dot = warp_sum(dot);
            if (lane == 0) scores[e] = dot;
        }
    }
    if (block_per_token) {
        __syncthreads();
        if (warp != 0) return;
    }
    __syncwarp();
    for (int x = lane; x < extra; x += 32) extra_out[static_cast<size_t>(token) * extra + x] = 1.0f / (1.0f + expf(-scores[experts + x]));
    if (bias != nullptr) {
        for (int e = lane; e < experts; e += 32) scores[e] += bias[e];
        __syncwarp();
    }
    if (score_kind == 2) {
        // the logits themselves rank the experts
    } else if (score_kind == 1) {
        float largest = -INFINITY;
        for (int e = lane; e < experts; e += 32) largest = fmaxf(largest, scores[e]);
        largest = warp_max(largest);
        float total = 0.0f;
        for (int e = lane; e < experts; e += 32) total += expf(scores[e] - largest);
        total = warp_sum(total);
        for (int e = lane; e < experts; e += 32) scores[e] = expf(scores[e] - largest) / total;
    } else {
        for (int e = lane; e < experts; e += 32) scores[e] = 1.0f / (1.0f + expf(-scores[e]));
    }
    __syncwarp();
    const int members = experts / group_count;
    for (int group = lane; group < group_count; group += 32) {
        float first = -INFINITY, second = -INFINITY;
        for (int m = 0; m < members; ++m) {
            const float s = scores[group * members + m] + (choice_bias != nullptr ? choice_bias[group * members + m] : 0.0f);
            if (s > first) {
                second = first;
                first = s;
            } else if (s > second) {
                second = s;
            }
        }
        group_score[group] = members >= 2 ? first + second : first;
    }
    for (int e = lane; e < experts; e += 32) candidates[e] = -INFINITY;
    __syncwarp();
    for (int round = 0; round < group_keep; ++round) {
        float best = -INFINITY;
        int best_group = 0x7fffffff;
        for (int group = lane; group < group_count; group += 32) {
            const float s = group_score[group];
            if (s > best) {   // ascending scan: the lowest index among equals stays
                best = s;
                best_group = group;
            }
        }
        warp_argmax(best, best_group);
        if (best_group == 0x7fffffff) break;
        for (int m = lane; m < members; m += 32)
            candidates[best_group * members + m] = scores[best_group * members + m] + (choice_bias != nullptr ? choice_bias[best_group * members + m] : 0.0f);
        if (lane == 0) group_score[best_group] = -INFINITY;
        __syncwarp();
    }
    float total = 0.0f;
    for (int round = 0; round < top; ++round) {
        float best = -INFINITY;
        int best_expert = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float s = candidates[e];
            if (s > best) {
                best = s;
                best_expert = e;
            }
        }
        warp_argmax(best, best_expert);
        if (best_expert == 0x7fffffff) best_expert = 0, best = 0.0f;   // fewer eligible experts than `top`: a weight of zero
        else if (choice_bias != nullptr) best = scores[best_expert];   // ranked with the bias, weighed without it
        total += best;
        if (lane == 0) {
            chosen[static_cast<size_t>(token) * top + round] = best_expert;
            weights[static_cast<size_t>(token) * top + round] = best;
            if (best_expert < experts) candidates[best_expert] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0 && renormalize == 2) {
        // the softmax over the chosen scores only (the first chosen is the largest)
        float* mine = weights + static_cast<size_t>(token) * top;
        const float largest = mine[0];
        float sum = 0.0f;
        for (int round = 0; round < top; ++round) {
            mine[round] = expf(mine[round] - largest);
            sum += mine[round];
        }
        for (int round = 0; round < top; ++round) mine[round] = mine[round] / sum * weight_scale;
    } else if (lane == 0) {
        const float factor = (renormalize && total > 0.0f ? 1.0f / total : 1.0f) * weight_scale;
        if (factor != 1.0f)
            for (int round = 0; round < top; ++round) weights[static_cast<size_t>(token) * top + round] *= factor;
    }
}

__device__ __forceinline__ float moe_activate(float v, int activation) {
    if (activation == 0) return v / (1.0f + expf(-v));                                   // silu
    if (activation == 1) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));    // gelu (exact)
    return v;
}

// The hidden value of a gated expert from its two 32-bit sums, as a value of T.
template <typename T>
__device__ __forceinline__ float moe_hidden(float gate, float up, int activation, float limit) {
    if (activation == kSigmoidLimit) return round_to<T>(sigmoid_limit_gate(gate, up, limit));
    return round_to<T>(round_to<T>(moe_activate(round_to<T>(gate), activation)) * round_to<T>(up));
}

// The hidden value of an expert without a gate, act(W_up x), from its 32-bit sum: activated in 32-bit, rounded once.
template <typename T>
__device__ __forceinline__ float moe_plain_hidden(float up, int activation) {
    return round_to<T>(moe_activate(up, activation));
}

// One block per (token, chosen expert) pair p (`gate` null: experts without a gate, hidden = act(W_up[e] x)): hidden = act(W_gate[e] x) * (W_up[e] x), rounded to T; out[p] = W_down[e] hidden
// in 32-bit.  A warp per output row, lanes along the row, sums in lane order then over the warp.
//   gate, up [experts, ff, width];  down [experts, width, ff];  out [pairs, width] (32-bit)
template <typename T>
__global__ void moe_expert_stream_kernel(const T* __restrict__ x, const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ down,
                                         const int* __restrict__ chosen, float* __restrict__ out, int top, int width, int ff, int experts,
                                         int activation, float limit) {
    extern __shared__ float shared[];
    float* x_s = shared;           // width
    float* hidden = shared + width;   // ff
    const int pair = blockIdx.x;
    const int token = pair / top;
    const int expert = chosen[pair];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* dst = out + static_cast<size_t>(pair) * width;
    if (expert < 0 || expert >= experts) {
        for (int d = threadIdx.x; d < width; d += blockDim.x) dst[d] = 0.0f;
        return;
    }
    for (int d = threadIdx.x; d < width; d += blockDim.x) x_s[d] = to_float(x[static_cast<size_t>(token) * width + d]);
    __syncthreads();
    const T* up_rows = up + static_cast<size_t>(expert) * ff * width;
    const T* gate_rows = gate != nullptr ? gate + static_cast<size_t>(expert) * ff * width : up_rows;
    for (int f = warp; f < ff; f += warps) {
        const T* g_row = gate_rows + static_cast<size_t>(f) * width;
        const T* u_row = up_rows + static_cast<size_t>(f) * width;
        float g = 0.0f, u = 0.0f;
        for (int d = lane; d < width; d += 32) {
            if (gate != nullptr) g += x_s[d] * to_float(g_row[d]);
            u += x_s[d] * to_float(u_row[d]);
        }
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) hidden[f] = gate != nullptr ? moe_hidden<T>(g, u, activation, limit) : moe_plain_hidden<T>(u, activation);
    }
    __syncthreads();
    const T* down_rows = down + static_cast<size_t>(expert) * width * ff;
    for (int r = warp; r < width; r += warps) {
        const T* d_row = down_rows + static_cast<size_t>(r) * ff;
        float sum = 0.0f;
        for (int f = lane; f < ff; f += 32) sum += hidden[f] * to_float(d_row[f]);
        sum = warp_sum(sum);
        if (lane == 0) dst[r] = sum;
    }
}

// out[t, :] = T(sum_k weights[t, k] * expert_out[t * top + k, :]), added in the order of k.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ expert_out, const float* __restrict__ weights, const int* __restrict__ chosen, int experts,
                                   T* __restrict__ out, int top, int width) {
    const int token = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int expert = chosen[static_cast<size_t>(token) * top + k];
            if (expert < 0 || expert >= experts) continue;   // no expert: nothing was computed for the pair
            sum += weights[static_cast<size_t>(token) * top + k] * expert_out[(static_cast<size_t>(token) * top + k) * width + d];
        }
        out[static_cast<size_t>(token) * width + d] = from_float<T>(sum);
    }
}

// residual[t, :] += sum_k weights[t, k] * expert_out[t * top + k, :] + every_gate[t] * every[t, :] on the 32-bit residual stream:
// the routed experts' weighted sum (in the order of k) and what every token runs besides (`every`, may be null; `every_gate`
// one 32-bit number per token, null: 1), added in 32-bit without a rounding in between.
template <typename T>
__global__ void moe_combine_add_kernel(const float* __restrict__ expert_out, const float* __restrict__ weights, const int* __restrict__ chosen, int experts,
                                       const T* __restrict__ every, const float* __restrict__ every_gate, int gate_stride, float* __restrict__ residual,
                                       int top, int width) {
    const int token = blockIdx.x;
    const float gate = every_gate != nullptr ? every_gate[static_cast<size_t>(token) * gate_stride] : 1.0f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int expert = chosen[static_cast<size_t>(token) * top + k];
            if (expert < 0 || expert >= experts) continue;
            sum += weights[static_cast<size_t>(token) * top + k] * expert_out[(static_cast<size_t>(token) * top + k) * width + d];
        }
        if (every != nullptr) sum += gate * to_float(every[static_cast<size_t>(token) * width + d]);
        residual[static_cast<size_t>(token) * width + d] += sum;
    }
}

// ---------------------------------------------------------------- few tokens: 16-byte loads, many blocks
// The same two products with the rows of an expert's matrices shared out over blocks: grid (pairs, row slices),
// four warps, a warp takes eight rows, four at a time, a lane 16 bytes of each row per turn (so eight loads of a
// lane are on their way at once).  Needs rows of 16-byte multiples.
constexpr int kStreamRowsPerWarp = 8, kStreamWarps = 4, kStreamRowsPerBlock = kStreamRowsPerWarp * kStreamWarps;

template <typename T, int V>
__device__ __forceinline__ void load_vector(const T* address, float (&values)[V]) {
    if constexpr (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(address);
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 two = __bfloat1622float2(pairs[i]);
            values[2 * i] = two.x;
            values[2 * i + 1] = two.y;
        }
    } else {
        const float4 raw = *reinterpret_cast<const float4*>(address);
        values[0] = raw.x, values[1] = raw.y, values[2] = raw.z, values[3] = raw.w;
    }
}

// sums[r] = x_s . rows[r], r < 4 (rows that do not exist are given as the first row and ignored by the caller)
template <typename T>
__device__ __forceinline__ void four_dots(const float* __restrict__ x_s, const T* const (&rows)[4], int length, int lane, float (&sums)[4]) {
    constexpr int V = 16 / sizeof(T);
#pragma unroll
    for (int r = 0; r < 4; ++r) sums[r] = 0.0f;
    for (int c = lane * V; c < length; c += 32 * V) {
        float w[4][V];
#pragma unroll
        for (int r = 0; r < 4; ++r) load_vector<T, V>(rows[r] + c, w[r]);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float xv = x_s[c + i];
#pragma unroll
            for (int r = 0; r < 4; ++r) sums[r] += xv * w[r][i];
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) sums[r] = warp_sum(sums[r]);
}

// hidden[pair, f] = T(act(gate[e][f] . x) * (up[e][f] . x)) for the block's slice of f (`gate` null: T(act(up[e][f] . x))).
template <typename T>
__global__ void __launch_bounds__(32 * kStreamWarps)
moe_gate_up_stream_kernel(const T* __restrict__ x, const T* __restrict__ gate, const T* __restrict__ up, const int* __restrict__ chosen,
                          T* __restrict__ hidden, int top, int width, int ff, int experts, int activation, float limit) {
    extern __shared__ float x_s[];   // width
    const int pair = blockIdx.x, token = pair / top, expert = chosen[pair];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = blockIdx.y * kStreamRowsPerBlock + warp * kStreamRowsPerWarp;
    if (expert < 0 || expert >= experts) {
        for (int f = first + lane; f < min(ff, first + kStreamRowsPerWarp); f += 32) hidden[static_cast<size_t>(pair) * ff + f] = from_float<T>(0.0f);
        return;
    }
    for (int d = threadIdx.x; d < width; d += blockDim.x) x_s[d] = to_float(x[static_cast<size_t>(token) * width + d]);
    __syncthreads();
    const T* up_rows = up + static_cast<size_t>(expert) * ff * width;
    const T* gate_rows = gate != nullptr ? gate + static_cast<size_t>(expert) * ff * width : up_rows;
    for (int f0 = first; f0 < min(ff, first + kStreamRowsPerWarp); f0 += 4) {
        const T* g_rows[4];
        const T* u_rows[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int f = f0 + r < ff ? f0 + r : f0;
            g_rows[r] = gate_rows + static_cast<size_t>(f) * width;
            u_rows[r] = up_rows + static_cast<size_t>(f) * width;
        }
        float g[4] = {0.0f, 0.0f, 0.0f, 0.0f}, u[4];
        if (gate != nullptr) four_dots<T>(x_s, g_rows, width, lane, g);
        four_dots<T>(x_s, u_rows, width, lane, u);
        if (lane < 4 && f0 + lane < ff) {
            const float gv = lane == 0 ? g[0] : lane == 1 ? g[1] : lane == 2 ? g[2] : g[3];
            const float uv = lane == 0 ? u[0] : lane == 1 ? u[1] : lane == 2 ? u[2] : u[3];
            hidden[static_cast<size_t>(pair) * ff + f0 + lane] = from_float<T>(gate != nullptr ? moe_hidden<T>(gv, uv, activation, limit) : moe_plain_hidden<T>(uv, activation));
        }
    }
}

// out[pair, r] = down[e][r] . hidden[pair] for the block's slice of r (32-bit).
template <typename T>
__global__ void __launch_bounds__(32 * kStreamWarps)
moe_down_stream_kernel(const T* __restrict__ hidden, const T* __restrict__ down, const int* __restrict__ chosen, float* __restrict__ out, int width,
                       int ff, int experts) {
    extern __shared__ float h_s[];   // ff
    const int pair = blockIdx.x, expert = chosen[pair];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = blockIdx.y * kStreamRowsPerBlock + warp * kStreamRowsPerWarp;
    float* dst = out + static_cast<size_t>(pair) * width;
    if (expert < 0 || expert >= experts) {
        for (int r = first + lane; r < min(width, first + kStreamRowsPerWarp); r += 32) dst[r] = 0.0f;
        return;
    }
    for (int f = threadIdx.x; f < ff; f += blockDim.x) h_s[f] = to_float(hidden[static_cast<size_t>(pair) * ff + f]);
    __syncthreads();
    const T* down_rows = down + static_cast<size_t>(expert) * width * ff;
    for (int r0 = first; r0 < min(width, first + kStreamRowsPerWarp); r0 += 4) {
        const T* rows[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) rows[r] = down_rows + static_cast<size_t>(r0 + r < width ? r0 + r : r0) * ff;
        float sums[4];
        four_dots<T>(h_s, rows, ff, lane, sums);
        if (lane < 4 && r0 + lane < width) dst[r0 + lane] = lane == 0 ? sums[0] : lane == 1 ? sums[1] : lane == 2 ? sums[2] : sums[3];
    }
}

// ---------------------------------------------------------------- many tokens: pairs grouped by expert, tensor cores
// Pairs sorted by expert: offsets[e] .. offsets[e + 1] are the places of expert e's pairs in `sorted` (pairs whose
// expert is no expert are left out).  One block; the order of an expert's pairs among themselves is whatever the
// shared-memory counters give, which changes no result: every pair's row is computed by itself.
__global__ void moe_sort_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ offsets, int* __restrict__ sorted) {
    extern __shared__ int counters[];   // experts counts, then experts cursors
    int* cursors = counters + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counters[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) atomicAdd(&counters[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = total;
            cursors[e] = total;
            total += counters[e];
        }
        offsets[experts] = total;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) sorted[atomicAdd(&cursors[e], 1)] = p;
    }
}

__device__ __forceinline__ void moe_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void moe_copy_16(void* shared_destination, const void* global_source, bool real) {
    if (real) {
        const uint32_t destination = static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(destination), "l"(global_source) : "memory");
    } else {
        *reinterpret_cast<uint4*>(shared_destination) = make_uint4(0u, 0u, 0u, 0u);
    }
}

constexpr int kGroupedM = 64, kGroupedN = 64, kGroupedK = 32, kGroupedPitch = kGroupedK + 8;   // bfloat16 elements; the pitch keeps fragment reads apart

// One tile of 64 sorted pairs of one expert times 64 output columns, K in steps of 32 through two stages of
// cp.async.  grid (tiles at most, column tiles); four warps of 16 rows each.
//   MODE 1 (gated):  A = x rows gathered by the pairs' tokens [.., K = width], B = gate[e] and up[e] [N = ff][K];
//           hidden[place, n] = T(act(A . gate[n]) * (A . up[n]))
//   MODE 2 (no gate):  A as above, B = up[e];   hidden[place, n] = T(act(A . up[n]))
//   MODE 0 (down):   A = hidden[place] [K = ff], B = down[e] [N = width][K];   out[pair, n] = A . down[n]  (32-bit)
template <int MODE>
__global__ void __launch_bounds__(128)
moe_grouped_kernel(const __nv_bfloat16* __restrict__ a_base, const __nv_bfloat16* __restrict__ b_first, const __nv_bfloat16* __restrict__ b_second,
                   const int* __restrict__ offsets, const int* __restrict__ sorted, __nv_bfloat16* __restrict__ hidden_out, float* __restrict__ pair_out,
                   int experts, int top, int n_total, int k_total, int activation, float limit) {
    constexpr bool GATED = MODE == 1, UP = MODE != 0;   // UP: rows gathered by token, hidden values out
    __shared__ __align__(16) __nv_bfloat16 a_s[2][kGroupedM][kGroupedPitch];
    __shared__ __align__(16) __nv_bfloat16 b_s[GATED ? 2 : 1][2][kGroupedN][kGroupedPitch];
    __shared__ int row_source[kGroupedM];   // GATED: the token of the row's pair; else: the pair itself; -1 past the expert's pairs
    __shared__ int tile_info[3];            // expert, first place, rows
    if (threadIdx.x == 0) {
        int expert = -1, first = 0, rows = 0, seen = 0;
        for (int e = 0; e < experts; ++e) {
            const int begin = offsets[e], count = offsets[e + 1] - begin;
            const int tiles = (count + kGroupedM - 1) / kGroupedM;
            if (static_cast<int>(blockIdx.x) < seen + tiles) {
                expert = e;
                first = begin + (static_cast<int>(blockIdx.x) - seen) * kGroupedM;
                rows = min(kGroupedM, begin + count - first);
                break;
            }
            seen += tiles;
        }
        tile_info[0] = expert, tile_info[1] = first, tile_info[2] = rows;
    }
    __syncthreads();
    const int expert = tile_info[0], first = tile_info[1], rows = tile_info[2];
    if (expert < 0) return;
    if (threadIdx.x < kGroupedM) {
        const int pair = static_cast<int>(threadIdx.x) < rows ? sorted[first + threadIdx.x] : -1;
        row_source[threadIdx.x] = pair < 0 ? -1 : (UP ? pair / top : pair);
    }
    __syncthreads();
    const int n0 = blockIdx.y * kGroupedN;
    const size_t b_expert = static_cast<size_t>(expert) * n_total * k_total;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    auto load_stage = [&](int stage, int k0) {
        // 64 rows x 4 chunks of 16 bytes per operand: two chunks a thread
        for (int index = threadIdx.x; index < kGroupedM * 4; index += 128) {
            const int row = index >> 2, chunk = index & 3, k = k0 + 8 * chunk;
            const bool in_k = k < k_total;
            const int source = row_source[row];
            const size_t a_row = UP ? static_cast<size_t>(source < 0 ? 0 : source) : static_cast<size_t>(first + row);
            moe_copy_16(&a_s[stage][row][8 * chunk], a_base + a_row * k_total + k, in_k && source >= 0);
            const bool in_n = n0 + row < n_total;
            const size_t b_row = b_expert + static_cast<size_t>(in_n ? n0 + row : 0) * k_total + k;
            moe_copy_16(&b_s[0][stage][row][8 * chunk], b_first + b_row, in_k && in_n);
            if constexpr (GATED) moe_copy_16(&b_s[1][stage][row][8 * chunk], b_second + b_row, in_k && in_n);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    float acc[GATED ? 2 : 1][kGroupedN / 8][4];
#pragma unroll
    for (int which = 0; which < (GATED ? 2 : 1); ++which)
#pragma unroll
        for (int j = 0; j < kGroupedN / 8; ++j) acc[which][j][0] = acc[which][j][1] = acc[which][j][2] = acc[which][j][3] = 0.0f;

    const int k_steps = (k_total + kGroupedK - 1) / kGroupedK;
    load_stage(0, 0);
    for (int step = 0; step < k_steps; ++step) {
        const int stage = step & 1;
        if (step + 1 < k_steps) {
            load_stage(stage ^ 1, (step + 1) * kGroupedK);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kGroupedK; kk += 16) {
            uint32_t a[4];
            a[0] = *reinterpret_cast<const uint32_t*>(&a_s[stage][16 * warp + g][kk + 2 * t]);
            a[1] = *reinterpret_cast<const uint32_t*>(&a_s[stage][16 * warp + g + 8][kk + 2 * t]);
            a[2] = *reinterpret_cast<const uint32_t*>(&a_s[stage][16 * warp + g][kk + 2 * t + 8]);
            a[3] = *reinterpret_cast<const uint32_t*>(&a_s[stage][16 * warp + g + 8][kk + 2 * t + 8]);
#pragma unroll
            for (int which = 0; which < (GATED ? 2 : 1); ++which) {
#pragma unroll
                for (int j = 0; j < kGroupedN / 8; ++j) {
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&b_s[which][stage][8 * j + g][kk + 2 * t]);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&b_s[which][stage][8 * j + g][kk + 2 * t + 8]);
                    moe_mma(acc[which][j], a, b0, b1);
                }
            }
        }
        __syncthreads();   // the stage is refilled in the turn after the next
    }
    // c[0], c[1]: row g, columns 2t and 2t + 1 of the 8-column tile; c[2], c[3]: row g + 8
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = 16 * warp + g + 8 * half;
        if (row >= rows) continue;
#pragma unroll
        for (int j = 0; j < kGroupedN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = n0 + 8 * j + 2 * t + e;
                if (n >= n_total) continue;
                if constexpr (GATED) {
                    using T = __nv_bfloat16;
                    const float gate_value = acc[0][j][2 * half + e], up_value = acc[1][j][2 * half + e];
                    hidden_out[static_cast<size_t>(first + row) * n_total + n] = from_float<T>(moe_hidden<T>(gate_value, up_value, activation, limit));
                } else if constexpr (UP) {
                    using T = __nv_bfloat16;
                    hidden_out[static_cast<size_t>(first + row) * n_total + n] = from_float<T>(moe_plain_hidden<T>(acc[0][j][2 * half + e], activation));
                } else {
                    pair_out[static_cast<size_t>(row_source[row]) * n_total + n] = acc[0][j][2 * half + e];
                }
            }
        }
    }
}

}  // namespace lb

extern "C" {

int lb_moe_route(const void* x, const float* router, int* chosen, float* weights, int tokens, int width, int experts, int top, int group_count,
                 int group_keep, int score_kind, int renormalize, float weight_scale, int dtype, cudaStream_t stream, const float* bias,
                 const float* choice_bias, int extra, float* extra_out) {
    // `router` has experts + extra rows; extra_out [tokens, extra] (see the kernel).
    if (tokens == 0) return 0;
    if (experts < 1 || top < 1 || top > experts || group_count < 1 || experts % group_count != 0 || group_keep < 1 || group_keep > group_count) return -2;
    if (extra < 0 || (extra > 0 && extra_out == nullptr)) return -2;
    constexpr int kWarps = 4;
    // A warp's scratch: scores, candidates, group scores (padded so that the staged row starts on 16 bytes), and the row.
    const int scratch = (2 * experts + extra + group_count + 3) / 4 * 4;
    if (static_cast<size_t>(kWarps) * scratch * sizeof(float) > 48 * 1024) return -2;
    int row_floats = width % 4 == 0 ? width : 0;   // rows of 16-byte multiples are staged and read 16 bytes a lane
    if (static_cast<size_t>(kWarps) * (scratch + row_floats) * sizeof(float) > 160 * 1024) row_floats = 0;
    const size_t shared = static_cast<size_t>(kWarps) * (scratch + row_floats) * sizeof(float);
    const int block_per_token = tokens <= 512 ? 1 : 0;   // few tokens: a block's warps share out a token's experts
    const int padded_groups = scratch - 2 * experts - extra;   // the kernel lays the three arrays out by these counts
    LB_DISPATCH_DTYPE(dtype, {
        auto kernel = lb::moe_route_kernel<T>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        kernel<<<block_per_token ? tokens : (tokens + kWarps - 1) / kWarps, 32 * kWarps, shared, stream>>>(
            static_cast<const T*>(x), router, chosen, weights, tokens, width, experts, top, group_count, group_keep, score_kind, renormalize, weight_scale,
            row_floats, padded_groups, bias, block_per_token, choice_bias, extra, extra_out);
    })
    return LB_LAUNCH_RESULT();
}

int lb_moe_expert_stream(const void* x, const void* gate, const void* up, const void* down, const int* chosen, float* out, int pairs, int top,
                         int width, int ff, int experts, int activation, int dtype, cudaStream_t stream, float limit) {
    if (pairs == 0) return 0;
    const size_t shared = (static_cast<size_t>(width) + ff) * sizeof(float);
    if (shared > 200 * 1024) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        auto kernel = lb::moe_expert_stream_kernel<T>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        kernel<<<pairs, 256, shared, stream>>>(static_cast<const T*>(x), static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<const T*>(down),
                                               chosen, out, top, width, ff, experts, activation, limit);
    })
    return LB_LAUNCH_RESULT();
}

int lb_moe_combine(const float* expert_out, const float* weights, const int* chosen, int experts, void* out, int tokens, int top, int width, int dtype,
                   cudaStream_t stream) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::moe_combine_kernel<T><<<tokens, 256, 0, stream>>>(expert_out, weights, chosen, experts, static_cast<T*>(out), top, width);
    })
    return LB_LAUNCH_RESULT();
}

int lb_moe_combine_add(const float* expert_out, const float* weights, const int* chosen, int experts, const void* every, const float* every_gate,
                       int gate_stride, float* residual, int tokens, int top, int width, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::moe_combine_add_kernel<T><<<tokens, 256, 0, stream>>>(expert_out, weights, chosen, experts, static_cast<const T*>(every), every_gate, gate_stride,
                                                                   residual, top, width);
    })
    return LB_LAUNCH_RESULT();
}

// The two products of the few-token path: `hidden` [pairs, ff] in the activation type, `out` [pairs, width] in 32-bit.
// Rows of 16-byte multiples only (width and ff multiples of 8 for bfloat16, of 4 for float32): -2 otherwise.
int lb_moe_expert_stream_wide(const void* x, const void* gate, const void* up, const void* down, const int* chosen, void* hidden, float* out, int pairs,
                              int top, int width, int ff, int experts, int activation, int dtype, cudaStream_t stream, float limit) {
    if (pairs == 0) return 0;
    const int vector = dtype == lb::kBFloat16 ? 8 : 4;
    if (width % vector != 0 || ff % vector != 0 || width * sizeof(float) > 160 * 1024 || ff * sizeof(float) > 160 * 1024) return -2;
    const dim3 up_grid(pairs, (ff + lb::kStreamRowsPerBlock - 1) / lb::kStreamRowsPerBlock), down_grid(pairs, (width + lb::kStreamRowsPerBlock - 1) / lb::kStreamRowsPerBlock);
    LB_DISPATCH_DTYPE(dtype, {
        auto first = lb::moe_gate_up_stream_kernel<T>;
        auto second = lb::moe_down_stream_kernel<T>;
        if (width * sizeof(float) > 48 * 1024) cudaFuncSetAttribute(first, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(width * sizeof(float)));
        if (ff * sizeof(float) > 48 * 1024) cudaFuncSetAttribute(second, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ff * sizeof(float)));
        first<<<up_grid, 32 * lb::kStreamWarps, width * sizeof(float), stream>>>(static_cast<const T*>(x), static_cast<const T*>(gate), static_cast<const T*>(up), chosen,
                                                                                static_cast<T*>(hidden), top, width, ff, experts, activation, limit);
        second<<<down_grid, 32 * lb::kStreamWarps, ff * sizeof(float), stream>>>(static_cast<const T*>(hidden), static_cast<const T*>(down), chosen, out, width, ff, experts);
    })
    return LB_LAUNCH_RESULT();
}

// The grouped path (bfloat16; width and ff multiples of 8; at most 1024 experts): sorts the pairs by expert into
// `offsets` [experts + 1] and `sorted` [pairs], then the two grouped products.  `hidden` is [pairs, ff] (rows in sorted
// order), `out` [pairs, width] in 32-bit (rows in pair order; rows of pairs without an expert are not written).
int lb_moe_experts_grouped(const void* x, const void* gate, const void* up, const void* down, const int* chosen, int* offsets, int* sorted, void* hidden,
                           float* out, int pairs, int top, int width, int ff, int experts, int activation, cudaStream_t stream, float limit) {
    if (pairs == 0) return 0;
    if (width % 8 != 0 || ff % 8 != 0 || experts < 1 || experts > 1024) return -2;
    lb::moe_sort_kernel<<<1, 1024, 2 * experts * sizeof(int), stream>>>(chosen, pairs, experts, offsets, sorted);
    const int tiles = (pairs + lb::kGroupedM - 1) / lb::kGroupedM + experts;   // no fewer than the experts' tiles together
    const auto* x16 = static_cast<const __nv_bfloat16*>(x);
    if (gate != nullptr)
        lb::moe_grouped_kernel<1><<<dim3(tiles, (ff + lb::kGroupedN - 1) / lb::kGroupedN), 128, 0, stream>>>(
            x16, static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), offsets, sorted, static_cast<__nv_bfloat16*>(hidden), nullptr, experts,
            top, ff, width, activation, limit);
    else
        lb::moe_grouped_kernel<2><<<dim3(tiles, (ff + lb::kGroupedN - 1) / lb::kGroupedN), 128, 0, stream>>>(
            x16, static_cast<const __nv_bfloat16*>(up), nullptr, offsets, sorted, static_cast<__nv_bfloat16*>(hidden), nullptr, experts, top, ff, width, activation,
            limit);
    lb::moe_grouped_kernel<0><<<dim3(tiles, (width + lb::kGroupedN - 1) / lb::kGroupedN), 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(hidden), static_cast<const __nv_bfloat16*>(down), nullptr, offsets, sorted, nullptr, out, experts, top, width, ff, activation, limit);
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
