// Embedding gather, RMS norm (with the residual sum fused in) and the gated activation.
//
// The residual stream is kept in 32-bit whatever the activation type is; the sum
// `residual + delta` and all norm statistics are computed in 32-bit.
#include "common.cuh"

namespace lb {

// residual[t, :] = float(table[ids[t], :]) * scale
// accumulate: residual[t, :] += ... instead (a model that feeds its input again further up)
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int dim, int vocab, float scale, int accumulate, int* status) {
    const int token = blockIdx.x;
    int id = ids[token];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report_error(status, kBadToken);
        id = 0;
    }
    const T* row = table + static_cast<size_t>(id) * dim;
    float* dst = out + static_cast<size_t>(token) * dim;
    if (accumulate) {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] += to_float(row[d]) * scale;
        return;
    }
    if (sizeof(T) == 2 && dim % 8 == 0) {
        // eight elements per thread and turn: one 16-byte load, two 16-byte stores
        for (int d = 8 * threadIdx.x; d < dim; d += 8 * blockDim.x) {
            const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(row) + d);
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 a = __bfloat1622float2(pairs[0]), b = __bfloat1622float2(pairs[1]), c = __bfloat1622float2(pairs[2]), e = __bfloat1622float2(pairs[3]);
            *reinterpret_cast<float4*>(dst + d) = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
            *reinterpret_cast<float4*>(dst + d + 4) = make_float4(c.x * scale, c.y * scale, e.x * scale, e.y * scale);
        }
        return;
    }
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = to_float(row[d]) * scale;
}

// One block per output row r.  src = rows ? rows[r] : r.
//   h = x[src] (+ delta[src]);   if write_back: x[src] = h  (x is the 32-bit residual stream)
//   n = T(h * rsqrt(mean(h^2) + eps));   out[r] = T(n * T(w + offset))
// The two roundings to T follow the reference's norm in its "only normalisation is upcast" mode; with `exact`
// the norm is 32-bit throughout, out[r] = T(h * rsqrt(..) * (w + offset)).
// With `slices` > 0 the delta is a product left as its K slices' partial sums: `partials[s][src][d]`, `slice_stride`
// floats apart, added in slice order and rounded to T as the product's own epilogue would have stored it.
template <typename TX, typename T>
__global__ void rmsnorm_kernel(TX* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ partials, int slices,
                               size_t slice_stride, const float* __restrict__ weight,
                               const int* __restrict__ rows, T* __restrict__ out, int dim, float eps,
                               float scale_offset, int write_back, int exact, const float* __restrict__ bias, int centred,
                               const float* __restrict__ delta_bias) {
    // bias (may be null): added to the output, out[r] = T(n * (w + offset) + bias).  centred: a layer norm,
    // n = (h - mean(h)) * rsqrt(mean((h - mean(h))^2) + eps), 32-bit throughout (taken with `exact`).
    // delta_bias (may be null; with a delta only): a 32-bit vector added to the delta, h = x + (delta + delta_bias).
    extern __shared__ float shared[];
    // Launched to start early: it is resident when the kernel before it ends (no launch in between).  Only then
    // may the product after it start and pull its weights towards L2: under the stream of the kernel before,
    // those weights would be gone again before they are read.
    wait_for_previous_kernel();
    allow_next_kernel();
    float* row_cache = shared;           // dim floats
    float* scratch = shared + dim;       // 33 floats
    const int r = blockIdx.x;
    const size_t src = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    TX* xr = x + src * dim;
    const T* dr = delta ? delta + src * dim : nullptr;
    const float* pr = slices > 0 ? partials + src * dim : nullptr;
    const bool adds = dr != nullptr || pr != nullptr;
    float sum = 0.0f;
    constexpr bool kVector = sizeof(TX) == 4 && sizeof(T) == 2;   // 32-bit stream in, bfloat16 out: four elements at a time
    if (kVector && dim % 4 == 0) {
        for (int d = 4 * threadIdx.x; d < dim; d += 4 * blockDim.x) {
            float4 h = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(xr) + d);
            if (dr) {
                const uint2 raw = *reinterpret_cast<const uint2*>(dr + d);
                const float2 low = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                const float2 high = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                h.x += low.x;
                h.y += low.y;
                h.z += high.x;
                h.w += high.y;
            }
            if (adds && delta_bias) {
                const float4 b = *reinterpret_cast<const float4*>(delta_bias + d);
                h.x += b.x;
                h.y += b.y;
                h.z += b.z;
                h.w += b.w;
            }
            if (pr) {
                // Four slices' loads leave before the first is added (the order of the additions stays).
                float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                int s = 0;
                for (; s + 4 <= slices; s += 4) {
                    float4 part[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) part[u] = __ldcs(reinterpret_cast<const float4*>(pr + static_cast<size_t>(s + u) * slice_stride + d));
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        total.x += part[u].x;
                        total.y += part[u].y;
                        total.z += part[u].z;
                        total.w += part[u].w;
                    }
                }
                for (; s < slices; ++s) {
                    const float4 part = __ldcs(reinterpret_cast<const float4*>(pr + static_cast<size_t>(s) * slice_stride + d));
                    total.x += part.x;
                    total.y += part.y;
                    total.z += part.z;
                    total.w += part.w;
                }
                h.x += round_to<T>(total.x);
                h.y += round_to<T>(total.y);
                h.z += round_to<T>(total.z);
                h.w += round_to<T>(total.w);
            }
            *reinterpret_cast<float4*>(row_cache + d) = h;
            sum += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float h = to_float(xr[d]);
            if (dr) h += to_float(dr[d]);
            if (adds && delta_bias) h += delta_bias[d];
            if (pr) {
                float total = 0.0f;
                for (int s = 0; s < slices; ++s) total += pr[static_cast<size_t>(s) * slice_stride + d];
                h += round_to<T>(total);
            }
            row_cache[d] = h;
            sum += h * h;
        }
    }
    T* dst = out + static_cast<size_t>(r) * dim;
    if (centred) {
        // the mean first, then the squared deviations from it (each thread rereads what it wrote)
        float plain = 0.0f;
        if (kVector && dim % 4 == 0) {
            for (int d = 4 * threadIdx.x; d < dim; d += 4 * blockDim.x) plain += (row_cache[d] + row_cache[d + 1]) + (row_cache[d + 2] + row_cache[d + 3]);
        } else {
            for (int d = threadIdx.x; d < dim; d += blockDim.x) plain += row_cache[d];
        }
        const float mean = block_sum(plain, scratch) / static_cast<float>(dim);
        float squares = 0.0f;
        if (kVector && dim % 4 == 0) {
            for (int d = 4 * threadIdx.x; d < dim; d += 4 * blockDim.x) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float c = row_cache[d + e] - mean;
                    squares += c * c;
                }
            }
        } else {
            for (int d = threadIdx.x; d < dim; d += blockDim.x) {
                const float c = row_cache[d] - mean;
                squares += c * c;
            }
        }
        const float inv_dev = rsqrtf(block_sum(squares, scratch) / static_cast<float>(dim) + eps);
        if (kVector && dim % 4 == 0) {
            for (int d = 4 * threadIdx.x; d < dim; d += 4 * blockDim.x) {
                const float4 h = *reinterpret_cast<const float4*>(row_cache + d);
                if (write_back && adds) *reinterpret_cast<float4*>(reinterpret_cast<float*>(xr) + d) = h;
                const float4 w = *reinterpret_cast<const float4*>(weight + d);
                const float4 b = bias ? *reinterpret_cast<const float4*>(bias + d) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                const __nv_bfloat162 low = __floats2bfloat162_rn((h.x - mean) * inv_dev * (w.x + scale_offset) + b.x, (h.y - mean) * inv_dev * (w.y + scale_offset) + b.y);
                const __nv_bfloat162 high = __floats2bfloat162_rn((h.z - mean) * inv_dev * (w.z + scale_offset) + b.z, (h.w - mean) * inv_dev * (w.w + scale_offset) + b.w);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&low);
                packed.y = *reinterpret_cast<const uint32_t*>(&high);
                *reinterpret_cast<uint2*>(dst + d) = packed;
            }
        } else {
            for (int d = threadIdx.x; d < dim; d += blockDim.x) {
                const float h = row_cache[d];
                if (write_back && adds) xr[d] = from_float<TX>(h);
                dst[d] = from_float<T>((h - mean) * inv_dev * (weight[d] + scale_offset) + (bias ? bias[d] : 0.0f));
            }
        }
        return;
    }
    const float total = block_sum(sum, scratch);
    const float inv = rsqrtf(total / static_cast<float>(dim) + eps);
    if (exact) {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            const float h = row_cache[d];
            if (write_back && adds) xr[d] = from_float<TX>(h);
            dst[d] = from_float<T>(h * inv * (weight[d] + scale_offset) + (bias ? bias[d] : 0.0f));
        }
    } else if (kVector && dim % 4 == 0) {
        for (int d = 4 * threadIdx.x; d < dim; d += 4 * blockDim.x) {
            const float4 h = *reinterpret_cast<const float4*>(row_cache + d);
            if (write_back && adds) *reinterpret_cast<float4*>(reinterpret_cast<float*>(xr) + d) = h;
            const float4 w = *reinterpret_cast<const float4*>(weight + d);
            const __nv_bfloat162 low = __floats2bfloat162_rn(round_to<T>(h.x * inv) * round_to<T>(w.x + scale_offset),
                                                             round_to<T>(h.y * inv) * round_to<T>(w.y + scale_offset));
            const __nv_bfloat162 high = __floats2bfloat162_rn(round_to<T>(h.z * inv) * round_to<T>(w.z + scale_offset),
                                                              round_to<T>(h.w * inv) * round_to<T>(w.w + scale_offset));
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t*>(&low);
            packed.y = *reinterpret_cast<const uint32_t*>(&high);
            *reinterpret_cast<uint2*>(dst + d) = packed;
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            const float h = row_cache[d];
            if (write_back && adds) xr[d] = from_float<TX>(h);
            const float n = round_to<T>(h * inv);
            const float w = round_to<T>(weight[d] + scale_offset);
            dst[d] = from_float<T>(n * w);
        }
    }
}

// x += delta on the 32-bit residual stream (used by norms that have no fused form).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t count) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) x[i] += to_float(delta[i]);
}

// out[r, :] = src[rows[r], :]
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows, T* __restrict__ out, int dim) {
    const size_t from = static_cast<size_t>(rows[blockIdx.x]) * dim, to = static_cast<size_t>(blockIdx.x) * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) out[to + d] = src[from + d];
}

__device__ __forceinline__ float activate(float v, int activation) {
    if (activation == 0) return v / (1.0f + expf(-v));                                   // silu
    if (activation == 1) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));    // gelu (exact)
    return v;                                                                            // identity
}

// fused[t] = [up (hidden) ; gate (hidden)];  out[t, f] = T(up * act(gate)), 32-bit inside.
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ fused, T* __restrict__ out, int hidden, size_t count,
                                        int activation, float limit) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const size_t token = i / hidden;
    const int f = static_cast<int>(i - token * hidden);
    const T* row = fused + token * 2 * static_cast<size_t>(hidden);
    const float up = to_float(row[f]);
    const float gate = to_float(row[hidden + f]);
    out[i] = activation == kSigmoidLimit ? from_float<T>(sigmoid_limit_gate(gate, up, limit)) : from_float<T>(up * round_to<T>(activate(gate, activation)));
}

// The same, eight elements per thread with 16-byte accesses (hidden % 8 == 0).
__global__ void gated_activation_bf16x8_kernel(const __nv_bfloat16* __restrict__ fused, __nv_bfloat16* __restrict__ out, int hidden,
                                               size_t groups, int activation, float limit) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const int per_row = hidden / 8;
    const size_t token = i / per_row;
    const int f = static_cast<int>(i - token * per_row) * 8;
    const __nv_bfloat16* row = fused + token * 2 * static_cast<size_t>(hidden);
    const uint4 up_raw = *reinterpret_cast<const uint4*>(row + f);
    const uint4 gate_raw = *reinterpret_cast<const uint4*>(row + hidden + f);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&up_raw);
    const __nv_bfloat162* gate = reinterpret_cast<const __nv_bfloat162*>(&gate_raw);
    uint4 result_raw;
    __nv_bfloat162* result = reinterpret_cast<__nv_bfloat162*>(&result_raw);
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
        const float2 u = __bfloat1622float2(up[pair]), g = __bfloat1622float2(gate[pair]);
        result[pair] = activation == kSigmoidLimit
                           ? __floats2bfloat162_rn(sigmoid_limit_gate(g.x, u.x, limit), sigmoid_limit_gate(g.y, u.y, limit))
                           : __floats2bfloat162_rn(u.x * round_to<__nv_bfloat16>(activate(g.x, activation)),
                                                   u.y * round_to<__nv_bfloat16>(activate(g.y, activation)));
    }
    *reinterpret_cast<uint4*>(out + token * static_cast<size_t>(hidden) + f) = result_raw;
}

// Fills one slot of every per-request state with a 32-bit pattern (zero at admission).  `table`
// holds, per state tensor, its base address and the bytes one slot takes; block (x, y) fills a
// piece of state y's slot.  States whose slots are 16-byte multiples are written 16 bytes at a time.
__global__ void fill_slots_kernel(const long long* __restrict__ table, int slot, unsigned pattern) {
    const long long base = table[2 * blockIdx.y], bytes = table[2 * blockIdx.y + 1];
    unsigned char* begin = reinterpret_cast<unsigned char*>(base) + static_cast<size_t>(slot) * bytes;
    const size_t first = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    if ((bytes % 16 == 0) && (base % 16 == 0)) {
        const uint4 value = make_uint4(pattern, pattern, pattern, pattern);
        for (size_t i = first; i < static_cast<size_t>(bytes) / 16; i += stride) reinterpret_cast<uint4*>(begin)[i] = value;
    } else {
        // odd sizes: byte by byte, the pattern's bytes in address order
        for (size_t i = first; i < static_cast<size_t>(bytes); i += stride) {
            const size_t address = reinterpret_cast<size_t>(begin) + i;
            begin[i] = static_cast<unsigned char>(pattern >> (8 * (address & 3)));
        }
    }
}

// Token ids that were sampled on the device in the step before and have not been to the host: the last
// token of segment s is taken from row source[s] of `sampled` (source[s] < 0: the host wrote it).
__global__ void feed_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ segment_start, const int* __restrict__ segment_length,
                                   const int* __restrict__ source, const int* __restrict__ sampled, int sampled_rows, int segments, int* status) {
    const int segment = blockIdx.x * blockDim.x + threadIdx.x;
    if (segment >= segments) return;
    const int row = source[segment];
    if (row < 0) return;
    if (row >= sampled_rows) {
        report_error(status, kBadToken);
        return;
    }
    token_ids[segment_start[segment] + segment_length[segment] - 1] = sampled[row];
}


// out[i] = T(x[i]): the 32-bit residual stream rounded to the activation type, for sublayers that read the
// stream itself and not a norm of it.
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, size_t count) {
    allow_next_kernel();   // a product launched to start early may ask for its weights meanwhile (it waits for this kernel's end before it reads)
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) out[i] = from_float<T>(x[i]);
}

// x[r, d] = T(x[r, d] + bias[d])
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int dim, size_t count) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) x[i] = from_float<T>(to_float(x[i]) + bias[i % dim]);
}

// The norm of a sublayer's output, added to the residual stream.  One block per row r:
//   y = scale_a * (a[r] + bias_a) + scale_b * (b[r] + bias_b)        (b and the biases may be absent; a may be given as the
//                                                                      un-summed outputs of a row's routed experts with their weights)
//   residual[r] += y * rsqrt(mean(y^2) + eps) * (w + offset)
//   rounded[r] = T(residual[r])                                      (if asked for: the next sublayer's input)
//   or, with next_weight: rounded[r] = T(residual[r] * rsqrt(mean(residual[r]^2) + next_eps) * (next_weight + next_offset)),
//   the norm that the next sublayer begins with
// Sum, statistics, norm and residual sum are 32-bit.
template <typename T>
__global__ void norm_accumulate_kernel(float* __restrict__ residual, const T* __restrict__ a, const float* __restrict__ bias_a, float scale_a,
                                       const T* __restrict__ b, const float* __restrict__ bias_b, float scale_b,
                                       const float* __restrict__ weight, T* __restrict__ rounded, int dim, float eps, float scale_offset,
                                       const float* __restrict__ next_weight, float next_eps, float next_offset,
                                       const float* __restrict__ pair_out, const float* __restrict__ pair_weight, const int* __restrict__ pair_expert,
                                       int top, int experts) {
    extern __shared__ float shared[];
    allow_next_kernel();   // as in cast_rows_kernel
    float* row_cache = shared;       // dim floats
    float* scratch = shared + dim;   // 33 floats
    const size_t base = static_cast<size_t>(blockIdx.x) * dim;
    float sum = 0.0f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float y;
        if (pair_out != nullptr) {
            // a is the weighted sum of a row's routed experts, left un-summed: added here in the order of the choice
            y = 0.0f;
            for (int k = 0; k < top; ++k) {
                const size_t pair = static_cast<size_t>(blockIdx.x) * top + k;
                const int expert = pair_expert[pair];
                if (expert >= 0 && expert < experts) y += pair_weight[pair] * pair_out[pair * dim + d];
            }
        } else {
            y = to_float(a[base + d]);
        }
        if (bias_a) y += bias_a[d];
        y *= scale_a;
        if (b) {
            float z = to_float(b[base + d]);
            if (bias_b) z += bias_b[d];
            y += scale_b * z;
        }
        row_cache[d] = y;
        sum += y * y;
    }
    const float total = block_sum(sum, scratch);
    const float inv = rsqrtf(total / static_cast<float>(dim) + eps);
    float squares = 0.0f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        const float h = residual[base + d] + row_cache[d] * inv * (weight[d] + scale_offset);
        residual[base + d] = h;
        if (next_weight) {
            row_cache[d] = h;   // each thread rereads only what it wrote
            squares += h * h;
        } else if (rounded) {
            rounded[base + d] = from_float<T>(h);
        }
    }
    if (next_weight == nullptr) return;
    const float next_inv = rsqrtf(block_sum(squares, scratch) / static_cast<float>(dim) + next_eps);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) rounded[base + d] = from_float<T>(row_cache[d] * next_inv * (next_weight[d] + next_offset));
}

// x[i] *= factor (32-bit, in place); with cap > 0 then x[i] = cap * tanh(x[i] / cap)
__global__ void scale_kernel(float* __restrict__ x, float factor, size_t count, float cap) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float v = x[i] * factor;
    x[i] = cap > 0.0f ? cap * tanhf(v / cap) : v;
}

// out[r, d] = T(act(x[r, d] + bias[d])) with the activation codes of the products' epilogues (bias may be null)
template <typename T>
__global__ void bias_activation_kernel(const T* __restrict__ x, const float* __restrict__ bias, T* __restrict__ out, int dim, size_t count, int activation) {
    allow_next_kernel();
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) out[i] = from_float<T>(activate(to_float(x[i]) + (bias ? bias[i % dim] : 0.0f), activation));
}

// out[t] = [T(stream[t]) | T(float(table[ids[t]]) * scale)]: the residual stream and the embedding's output side by
// side, rounded to the activation type, as the input of a projection that renews the stream from both.
template <typename T>
__global__ void stream_concat_kernel(const float* __restrict__ stream, const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out,
                                     int dim, int vocab, float scale, int* status) {
    allow_next_kernel();
    const int token = blockIdx.x;
    int id = ids[token];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report_error(status, kBadToken);
        id = 0;
    }
    const float* src = stream + static_cast<size_t>(token) * dim;
    const T* row = table + static_cast<size_t>(id) * dim;
    T* dst = out + static_cast<size_t>(token) * 2 * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        dst[d] = from_float<T>(src[d]);
        dst[dim + d] = from_float<T>(to_float(row[d]) * scale);
    }
}

// residual[r, :] += scale_a * rms_norm(a[r, :]) * weight_a + scale_b * rms_norm(b[r, :]) * weight_b on the 32-bit residual
// stream, everything in 32-bit (b may be null): the outputs of mixers that run side by side, each normed over the
// model's width under a weight of its own, then summed.  One block per row.
template <typename T>
__global__ void branch_norms_accumulate_kernel(float* __restrict__ residual, const T* __restrict__ a, const float* __restrict__ weight_a, float scale_a,
                                               const T* __restrict__ b, const float* __restrict__ weight_b, float scale_b, int dim, float eps) {
    __shared__ float scratch[33];
    const size_t row = static_cast<size_t>(blockIdx.x) * dim;
    float sum_a = 0.0f, sum_b = 0.0f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        const float va = to_float(a[row + d]);
        sum_a += va * va;
        if (b != nullptr) {
            const float vb = to_float(b[row + d]);
            sum_b += vb * vb;
        }
    }
    const float inv_a = rsqrtf(block_sum(sum_a, scratch) / static_cast<float>(dim) + eps);
    const float inv_b = b != nullptr ? rsqrtf(block_sum(sum_b, scratch) / static_cast<float>(dim) + eps) : 0.0f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float sum = scale_a * (to_float(a[row + d]) * inv_a * weight_a[d]);
        if (b != nullptr) sum += scale_b * (to_float(b[row + d]) * inv_b * weight_b[d]);
        residual[row + d] += sum;
    }
}

}  // namespace lb

extern "C" {

int lb_feed_tokens(int* token_ids, const int* segment_start, const int* segment_length, const int* source, const int* sampled, int sampled_rows,
                   int segments, int* status, cudaStream_t stream) {
    if (segments == 0) return 0;
    lb::feed_tokens_kernel<<<(segments + 127) / 128, 128, 0, stream>>>(token_ids, segment_start, segment_length, source, sampled, sampled_rows, segments, status);
    return LB_LAUNCH_RESULT();
}

// table: device array of `states` records (base address, bytes per slot), int64 each.
int lb_fill_slots(const long long* table, int states, long long largest_bytes, int slot, unsigned pattern, cudaStream_t stream) {
    if (states == 0 || largest_bytes == 0) return 0;
    long long pieces = (largest_bytes / 16 + 255) / 256;
    if (pieces < 1) pieces = 1;
    if (pieces > 64) pieces = 64;
    lb::fill_slots_kernel<<<dim3(static_cast<unsigned>(pieces), static_cast<unsigned>(states)), 256, 0, stream>>>(table, slot, pattern);
    return LB_LAUNCH_RESULT();
}

int lb_embed(const void* table, const int* ids, float* out, int tokens, int dim, int vocab, float scale, int dtype,
             int* status, cudaStream_t stream, int accumulate) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::embed_kernel<T><<<tokens, 256, 0, stream>>>(static_cast<const T*>(table), ids, out, dim, vocab, scale, accumulate, status);
    })
    return LB_LAUNCH_RESULT();
}

// x_is_float: 1 when x is the 32-bit residual stream, 0 when x has the activation type.
// partials, slices, slice_stride: see rmsnorm_kernel (slices == 0: none); the vector path needs slice_stride % 4 == 0.
int lb_rmsnorm(void* x, int x_is_float, const void* delta, const float* partials, int slices, long long slice_stride, const float* weight,
               const int* rows, void* out, int out_rows, int dim, float eps, float scale_offset, int write_back, int dtype, cudaStream_t stream,
               int exact, const float* bias, int centred, const float* delta_bias) {
    if (out_rows == 0) return 0;
    if ((bias != nullptr || centred) && !exact) return -2;   // an output bias and the layer norm exist in the 32-bit form only
    if (slices < 0 || (slices > 0 && (partials == nullptr || slice_stride < 0 || (dim % 4 == 0 && slice_stride % 4 != 0)))) return -2;
    const size_t shared = (static_cast<size_t>(dim) + 33) * sizeof(float);
    if (shared > 200 * 1024) return -2;
    // Few rows (decoding): the kernel is one trip to memory long if every thread has one piece of
    // the row, so a thread per four elements; many rows: 256 threads keep more rows resident per SM.
    int threads = dim >= 1024 ? 256 : 128;
    if (out_rows <= 64) {
        threads = ((dim + 3) / 4 + 31) / 32 * 32;
        threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
    }
    LB_DISPATCH_DTYPE(dtype, {
        if (x_is_float) {
            auto kernel = lb::rmsnorm_kernel<float, T>;
            if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
            lb::launch_overlapped(kernel, dim3(out_rows), dim3(threads), shared, stream, static_cast<float*>(x), static_cast<const T*>(delta), partials, slices,
                                  static_cast<size_t>(slice_stride), weight, rows, static_cast<T*>(out), dim, eps, scale_offset, write_back, exact, bias, centred, delta_bias);
        } else {
            auto kernel = lb::rmsnorm_kernel<T, T>;
            if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
            lb::launch_overlapped(kernel, dim3(out_rows), dim3(threads), shared, stream, static_cast<T*>(x), static_cast<const T*>(delta), partials, slices,
                                  static_cast<size_t>(slice_stride), weight, rows, static_cast<T*>(out), dim, eps, scale_offset, write_back, exact, bias, centred, delta_bias);
        }
    })
    return LB_LAUNCH_RESULT();
}

int lb_residual_add(float* x, const void* delta, long long count, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        lb::residual_add_kernel<T><<<blocks, 256, 0, stream>>>(x, static_cast<const T*>(delta), static_cast<size_t>(count));
    })
    return LB_LAUNCH_RESULT();
}

// element_size: 2 or 4 bytes per element (rows are copied bit for bit).
int lb_gather_rows(const void* src, const int* rows, void* out, int out_rows, int dim, int element_size,
                   cudaStream_t stream) {
    if (out_rows == 0) return 0;
    if (element_size == 4) {
        lb::gather_rows_kernel<float><<<out_rows, 256, 0, stream>>>(static_cast<const float*>(src), rows, static_cast<float*>(out), dim);
    } else if (element_size == 2) {
        lb::gather_rows_kernel<__nv_bfloat16><<<out_rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), rows,
                                                                           static_cast<__nv_bfloat16*>(out), dim);
    } else {
        return -1;
    }
    return LB_LAUNCH_RESULT();
}

int lb_gated_activation(const void* fused, void* out, int tokens, int hidden, int activation, int dtype,
                        cudaStream_t stream, float limit) {
    const size_t count = static_cast<size_t>(tokens) * hidden;
    if (count == 0) return 0;
    if (dtype == lb::kBFloat16 && hidden % 8 == 0) {
        const size_t groups = count / 8;
        lb::gated_activation_bf16x8_kernel<<<static_cast<unsigned>((groups + 255) / 256), 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(fused), static_cast<__nv_bfloat16*>(out), hidden, groups, activation, limit);
        return LB_LAUNCH_RESULT();
    }
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        lb::gated_activation_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T*>(fused), static_cast<T*>(out), hidden, count, activation, limit);
    })
    return LB_LAUNCH_RESULT();
}

int lb_cast_rows(const float* x, void* out, long long count, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        lb::cast_rows_kernel<T><<<blocks, 256, 0, stream>>>(x, static_cast<T*>(out), static_cast<size_t>(count));
    })
    return LB_LAUNCH_RESULT();
}

int lb_add_bias(void* x, const float* bias, int rows, int dim, int dtype, cudaStream_t stream) {
    const size_t count = static_cast<size_t>(rows) * dim;
    if (count == 0) return 0;
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        lb::add_bias_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<T*>(x), bias, dim, count);
    })
    return LB_LAUNCH_RESULT();
}

// b, bias_a, bias_b and rounded may be null.
int lb_norm_accumulate(float* residual, const void* a, const float* bias_a, float scale_a, const void* b, const float* bias_b, float scale_b,
                       const float* weight, void* rounded, int rows, int dim, float eps, float scale_offset, int dtype, cudaStream_t stream,
                       const float* next_weight, float next_eps, float next_offset, const float* pair_out, const float* pair_weight,
                       const int* pair_expert, int top, int experts) {
    if (next_weight != nullptr && rounded == nullptr) return -2;
    if (pair_out != nullptr && (pair_weight == nullptr || pair_expert == nullptr || top < 1)) return -2;
    if (rows == 0) return 0;
    const size_t shared = (static_cast<size_t>(dim) + 33) * sizeof(float);
    if (shared > 200 * 1024) return -2;
    int threads = ((dim + 3) / 4 + 31) / 32 * 32;
    threads = threads < 128 ? 128 : (threads > 512 ? 512 : threads);
    LB_DISPATCH_DTYPE(dtype, {
        auto kernel = lb::norm_accumulate_kernel<T>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        kernel<<<rows, threads, shared, stream>>>(residual, static_cast<const T*>(a), bias_a, scale_a, static_cast<const T*>(b), bias_b, scale_b, weight,
                                                  static_cast<T*>(rounded), dim, eps, scale_offset, next_weight, next_eps, next_offset, pair_out, pair_weight, pair_expert, top,
                                                  experts);
    })
    return LB_LAUNCH_RESULT();
}

// b and weight_b may be null (one branch).
int lb_branch_norms_accumulate(float* residual, const void* a, const float* weight_a, float scale_a, const void* b, const float* weight_b, float scale_b,
                               int rows, int dim, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (b != nullptr && weight_b == nullptr) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        lb::branch_norms_accumulate_kernel<T><<<rows, 256, 0, stream>>>(residual, static_cast<const T*>(a), weight_a, scale_a, static_cast<const T*>(b), weight_b,
                                                                         scale_b, dim, eps);
    })
    return LB_LAUNCH_RESULT();
}

int lb_scale(float* x, float factor, long long count, cudaStream_t stream, float cap) {
    if (count == 0) return 0;
    lb::scale_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, stream>>>(x, factor, static_cast<size_t>(count), cap);
    return LB_LAUNCH_RESULT();
}

int lb_bias_activation(const void* x, const float* bias, void* out, int rows, int dim, int activation, int dtype, cudaStream_t stream) {
    const size_t count = static_cast<size_t>(rows) * dim;
    if (count == 0) return 0;
    if (activation < 0 || activation > 2) return -2;
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        lb::bias_activation_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T*>(x), bias, static_cast<T*>(out), dim, count, activation);
    })
    return LB_LAUNCH_RESULT();
}

int lb_stream_concat(const float* stream_rows, const void* table, const int* ids, void* out, int tokens, int dim, int vocab, float scale, int dtype,
                     int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::stream_concat_kernel<T><<<tokens, 256, 0, stream>>>(stream_rows, static_cast<const T*>(table), ids, static_cast<T*>(out), dim, vocab, scale, status);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
