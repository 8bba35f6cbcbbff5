// The gated delta rule with one decay per head and key channel, over ragged portions of requests:
//
//   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// with S a [key_dim, value_dim] matrix per request and head, kept in 32-bit in the request's state
// slot.  Four kernels: `prepare` (short causal convolutions with silu over q, k and v, unit q and k,
// beta and the decays, all in 32-bit), `conv_state` (the convolutions' last inputs into the slot),
// `scan` (the recurrence, token by token) and `output` (per-head RMS norm times a sigmoid gate).
// The order of every sum depends on the token's place in its request only, never on how the
// request was cut into steps or on what else is in the batch.
#include "common.cuh"

#include <type_traits>

namespace lb {

constexpr int kPrepareMaxPerLane = 16;   // key_dim <= 512

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// The convolution's input of channel `ch` at relative time `rel` of the token's portion (negative: from the state,
// whose rows hold relative times -(taps-1) .. -1).
template <typename T>
__device__ __forceinline__ float conv_input(const T* __restrict__ proj, int proj_width, const T* __restrict__ state_rows, int channels,
                                            int start, int rel, int taps, int ch) {
    if (rel >= 0) return to_float(proj[static_cast<size_t>(start + rel) * proj_width + ch]);
    const int row = taps - 1 + rel;
    return row >= 0 ? to_float(state_rows[static_cast<size_t>(row) * channels + ch]) : 0.0f;
}

// y = silu(sum_j w[ch, taps-1-j] * input(t - j)), lags in the order j = 0, 1, ...  (Loading up to eight taps into
// registers before the first is used, under predicates, took 89 us where this loop takes 48.)
template <typename T>
__device__ __forceinline__ float conv_silu(const T* __restrict__ proj, int proj_width, const T* __restrict__ state_rows, int channels,
                                           const float* __restrict__ weight, int start, int rel, int taps, int ch) {
    float acc = 0.0f;
    for (int j = 0; j < taps; ++j)
        acc += weight[static_cast<size_t>(ch) * taps + (taps - 1 - j)] * conv_input(proj, proj_width, state_rows, channels, start, rel - j, taps, ch);
    return acc * sigmoidf_(acc);
}

// grid (tokens, slices of a token's units), a warp per unit: the `groups` query heads, the `groups` key heads, the
// `heads` value heads, and per head its decays and beta.
//   proj [tokens, proj_width]: q (groups x dk) | k (groups x dk) | v (heads x dv) | b (heads) | unused
//   ag   [tokens, ag_width]:   a (heads x dk) | ...
//   q_out, k_out [tokens, groups, dk], v_out [tokens, heads, dv], beta_out [tokens, heads], g_out [tokens, heads, dk]: 32-bit
template <typename T, bool UPDATE>
__global__ void gdr_prepare_kernel(const T* __restrict__ proj, int proj_width, const T* __restrict__ ag, int ag_width,
                                   std::conditional_t<UPDATE, T*, const T* __restrict__> conv_state, const float* __restrict__ conv_weight,
                                   const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out,
                                   float* __restrict__ beta_out, float* __restrict__ g_out,
                                   const int* __restrict__ token_segment, const int* __restrict__ segment_start,
                                   const int* __restrict__ segment_slot, int heads, int groups, int dk, int dv, int taps,
                                   int num_slots, float unit_eps, float q_scale, int* status, int decay_per_head) {
    // decay_per_head: `ag` holds one decay logit per head (heads columns) and dt_bias one element per head; the head's
    // decay is written to all of its key channels.
    // UPDATE: every portion of the step is one token, and the lane that convolves a channel (the only reader of that
    // channel's rows in the slot) also shifts the rows and appends the token's input; no state kernel runs after this one.
    // (Otherwise the state is read-only here, and says so: the loads were a third slower without it.)
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int segment = token_segment[token];
    const int start = segment_start[segment];
    const int slot = segment_slot[segment];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) report_error(status, kBadSlot);
        return;
    }
    const int channels = 2 * groups * dk + heads * dv;
    auto state_rows = conv_state + static_cast<size_t>(slot) * (taps > 1 ? taps - 1 : 0) * channels;
    const int rel = token - start;
    auto shift_state = [&](int ch) {
        if constexpr (UPDATE) {
            if (taps <= 1) return;
            for (int i = 0; i + 2 < taps; ++i) state_rows[static_cast<size_t>(i) * channels + ch] = state_rows[static_cast<size_t>(i + 1) * channels + ch];
            state_rows[static_cast<size_t>(taps - 2) * channels + ch] = proj[static_cast<size_t>(token) * proj_width + ch];
        }
    };
    const int units = 2 * groups + 2 * heads;
    for (int unit = blockIdx.y * warps + warp; unit < units; unit += gridDim.y * warps) {
        if (unit < 2 * groups) {
            // a query or key head: convolution, silu, unit length (and the query's scale)
            const bool is_query = unit < groups;
            const int head = is_query ? unit : unit - groups;
            const int ch0 = unit * dk;   // q channels come first, then k
            float values[kPrepareMaxPerLane];
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < kPrepareMaxPerLane; ++i) {
                const int c = lane + 32 * i;
                values[i] = 0.0f;
                if (c < dk) {
                    values[i] = conv_silu(proj, proj_width, state_rows, channels, conv_weight, start, rel, taps, ch0 + c);
                    sum += values[i] * values[i];
                    shift_state(ch0 + c);
                }
            }
            sum = warp_sum(sum);
            const float inv = rsqrtf(sum + unit_eps) * (is_query ? q_scale : 1.0f);
            float* dst = (is_query ? q_out : k_out) + (static_cast<size_t>(token) * groups + head) * dk;
#pragma unroll
            for (int i = 0; i < kPrepareMaxPerLane; ++i) {
                const int c = lane + 32 * i;
                if (c < dk) dst[c] = values[i] * inv;
            }
        } else if (unit < 2 * groups + heads) {
            const int head = unit - 2 * groups;
            const int ch0 = 2 * groups * dk + head * dv;
            float* dst = v_out + (static_cast<size_t>(token) * heads + head) * dv;
            for (int c = lane; c < dv; c += 32) {
                dst[c] = conv_silu(proj, proj_width, state_rows, channels, conv_weight, start, rel, taps, ch0 + c);
                shift_state(ch0 + c);
            }
        } else {
            const int head = unit - 2 * groups - heads;
            const float rate = expf(a_log[head]);
            const T* a_row = ag + static_cast<size_t>(token) * ag_width + static_cast<size_t>(head) * dk;
            float* dst = g_out + (static_cast<size_t>(token) * heads + head) * dk;
            if (decay_per_head) {
                const float decay = expf(-rate * softplusf_(to_float(ag[static_cast<size_t>(token) * ag_width + head]) + dt_bias[head]));
                for (int c = lane; c < dk; c += 32) dst[c] = decay;
            } else {
                for (int c = lane; c < dk; c += 32) dst[c] = expf(-rate * softplusf_(to_float(a_row[c]) + dt_bias[head * dk + c]));
            }
            if (lane == 0) beta_out[static_cast<size_t>(token) * heads + head] = sigmoidf_(to_float(proj[static_cast<size_t>(token) * proj_width + channels + head]));
        }
    }
}

// grid (portions, channel slices): the slot's rows become the last taps-1 inputs of [old rows ; the portion's inputs].
// A thread walks a channel's rows upwards; row i is written after row length + i (> i) was read.
template <typename T>
__global__ void gdr_conv_state_kernel(const T* __restrict__ proj, int proj_width, T* __restrict__ conv_state, const int* __restrict__ segment_start,
                                      const int* __restrict__ segment_length, const int* __restrict__ segment_slot, int channels, int taps,
                                      int num_slots) {
    const int segment = blockIdx.x;
    const int slot = segment_slot[segment];
    if (slot < 0 || slot >= num_slots) return;   // reported by the kernel before
    const int start = segment_start[segment], length = segment_length[segment];
    T* rows = conv_state + static_cast<size_t>(slot) * (taps - 1) * channels;
    for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
        for (int i = 0; i < taps - 1; ++i) {
            const int rel = length - (taps - 1) + i;
            rows[static_cast<size_t>(i) * channels + ch] =
                rel >= 0 ? proj[static_cast<size_t>(start + rel) * proj_width + ch] : rows[static_cast<size_t>(taps - 1 + rel) * channels + ch];
        }
    }
}

// The recurrence.  grid (portions, heads, ceil(dv / 8)); a block holds 8 columns of S, a thread R = 8 rows of one
// column in registers.  A column's DKP rows (key_dim rounded up, padded rows stay zero) are spread over SPLIT = DKP / 8
// neighbouring lanes; lane `part` holds the rows ((i / 4) * SPLIT + part) * 4 + i % 4, so that the lanes of a column read
// neighbouring 16-byte pieces of k, q and g from shared memory.  A token's step is one chain of dependent instructions
// (decay, dot, the lanes' sums, write, read-out, the lanes' sums) that a warp issues in order, and a multiprocessor's
// schedulers hold one warp each here, which issues about one instruction in three cycles: so the kernel is as fast as a
// warp's instructions per token are few, hence many small blocks (a sequence of 2,048 tokens at 8 heads of 64 x 128
// runs on 128 blocks of two warps).  Measured at those sizes: 32 rows x 1 column a lane 304 ns a token, 8 rows x 4
// columns 382 ns, 8 rows x 1 column 273 ns.  Tokens come in batches through two stages of shared memory: the next
// batch's k, q, g, v and beta are on their way (cp.async) while this one is worked on.  Every sum runs in a fixed order.
constexpr int kScanCols = 8, kScanThreadCols = 1, kScanThreadRows = 8;

template <int DKP>
struct ScanShared {
    static constexpr int kBatch = 8;   // small stages: many blocks fit a multiprocessor, whose warps hide each other's waits
    static constexpr int kStageFloats = kBatch * (3 * DKP + kScanCols + 4);   // k, q, g rows, v columns, beta (padded to 16 bytes)
    static constexpr size_t kBytes = 2 * kStageFloats * sizeof(float);
};

__device__ __forceinline__ void scan_copy_4(float* shared_destination, const float* global_source) {
    const uint32_t destination = static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(destination), "l"(global_source) : "memory");
}
__device__ __forceinline__ void scan_copy_16(float* shared_destination, const float* global_source) {
    const uint32_t destination = static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(destination), "l"(global_source) : "memory");
}

// DELTA false: the plain linear recurrence S <- diag(g_t) S + k_t v_t^T, o_t = S^T q_t (no correction by what the state
// already holds under k_t, no beta): the same state layout, stages and read-out with a shorter chain per token.
template <int DKP, int SPLIT, bool DELTA>
__global__ void __launch_bounds__((kScanCols / kScanThreadCols) * SPLIT)
gdr_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ g, const float* __restrict__ v,
                const float* __restrict__ beta, float* __restrict__ state, float* __restrict__ out, const int* __restrict__ segment_start,
                const int* __restrict__ segment_length, const int* __restrict__ segment_slot, int heads, int groups, int dk, int dv,
                int num_slots, int* status, const int* __restrict__ segment_list, int v_columns) {
    // segment_list (may be null): the portions this launch runs.  v_columns <= dv: the columns `v` really has (rows of
    // heads x v_columns); the columns past them get zeros as values (they carry a transition matrix, see the chunked path).
    constexpr int R = kScanThreadRows, C = kScanThreadCols;
    static_assert(DKP == R * SPLIT && SPLIT <= 32, "a column's rows lie in one warp");
    using Shared = ScanShared<DKP>;
    constexpr int kBatch = Shared::kBatch;
    extern __shared__ __align__(16) float scan_memory[];
    const int segment = segment_list ? segment_list[blockIdx.x] : static_cast<int>(blockIdx.x);
    const int head = blockIdx.y, col0 = blockIdx.z * kScanCols;
    const int tid = threadIdx.x, column_group = tid / SPLIT, part = tid % SPLIT;
    const int group = head / (heads / groups);
    const int slot = segment_slot[segment];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) report_error(status, kBadSlot);
        return;
    }
    const int start = segment_start[segment], length = segment_length[segment];
    const int column = col0 + C * column_group;   // the thread's first column
    auto k_of = [&](int stage) { return scan_memory + stage * Shared::kStageFloats; };
    auto q_of = [&](int stage) { return k_of(stage) + kBatch * DKP; };
    auto g_of = [&](int stage) { return k_of(stage) + 2 * kBatch * DKP; };
    auto v_of = [&](int stage) { return k_of(stage) + 3 * kBatch * DKP; };
    auto beta_of = [&](int stage) { return v_of(stage) + kBatch * kScanCols; };
    // The padding (rows of S past key_dim, columns past value_dim) is written once: the copies never touch it.
    for (int index = tid; index < 2 * kBatch * DKP; index += blockDim.x) {
        const int stage = index / (kBatch * DKP), rest = index - stage * kBatch * DKP;
        if (rest % DKP >= dk) {
            k_of(stage)[rest] = 0.0f;
            q_of(stage)[rest] = 0.0f;
            g_of(stage)[rest] = 1.0f;
        }
    }
    for (int index = tid; index < 2 * kBatch * kScanCols; index += blockDim.x) {
        const int stage = index / (kBatch * kScanCols), rest = index - stage * kBatch * kScanCols;
        if (col0 + rest % kScanCols >= v_columns) v_of(stage)[rest] = 0.0f;
    }
    const bool wide = dk % 4 == 0;   // rows of 16-byte multiples (the buffers are 16-byte aligned)
    auto fetch = [&](int stage, int t0) {
        const int n = min(kBatch, length - t0);
        if (wide) {
            const int pieces = dk / 4;
            for (int index = tid; index < n * pieces; index += blockDim.x) {
                const int tt = index / pieces, c = 4 * (index - tt * pieces);
                const size_t token = static_cast<size_t>(start + t0 + tt);
                scan_copy_16(k_of(stage) + tt * DKP + c, k + (token * groups + group) * dk + c);
                scan_copy_16(q_of(stage) + tt * DKP + c, q + (token * groups + group) * dk + c);
                scan_copy_16(g_of(stage) + tt * DKP + c, g + (token * heads + head) * dk + c);
            }
        } else {
            for (int index = tid; index < n * dk; index += blockDim.x) {
                const int tt = index / dk, c = index - tt * dk;
                const size_t token = static_cast<size_t>(start + t0 + tt);
                scan_copy_4(k_of(stage) + tt * DKP + c, k + (token * groups + group) * dk + c);
                scan_copy_4(q_of(stage) + tt * DKP + c, q + (token * groups + group) * dk + c);
                scan_copy_4(g_of(stage) + tt * DKP + c, g + (token * heads + head) * dk + c);
            }
        }
        const int columns = min(kScanCols, v_columns - col0);
        for (int index = tid; index < n * columns; index += blockDim.x) {
            const int tt = index / columns, c = index - tt * columns;
            scan_copy_4(v_of(stage) + tt * kScanCols + c, v + (static_cast<size_t>(start + t0 + tt) * heads + head) * v_columns + col0 + c);
        }
        if constexpr (DELTA)
            for (int tt = tid; tt < n; tt += blockDim.x) scan_copy_4(beta_of(stage) + tt, beta + static_cast<size_t>(start + t0 + tt) * heads + head);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    fetch(0, 0);
    float* S_base = state + (static_cast<size_t>(slot) * heads + head) * dk * dv;
    float S[C][R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = ((i >> 2) * SPLIT + part) * 4 + (i & 3);
#pragma unroll
        for (int c = 0; c < C; ++c) S[c][i] = (row < dk && column + c < dv) ? S_base[static_cast<size_t>(row) * dv + column + c] : 0.0f;
    }
    int stage = 0;
    for (int t0 = 0; t0 < length; t0 += kBatch, stage ^= 1) {
        const int n = min(kBatch, length - t0);
        if (t0 + kBatch < length) {
            fetch(stage ^ 1, t0 + kBatch);   // that stage was used up in the turn before (the barrier at its end)
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const float* beta_s = beta_of(stage);
        for (int tt = 0; tt < n; ++tt) {
            const float4* k4 = reinterpret_cast<const float4*>(k_of(stage) + tt * DKP);
            const float4* q4 = reinterpret_cast<const float4*>(q_of(stage) + tt * DKP);
            const float4* g4 = reinterpret_cast<const float4*>(g_of(stage) + tt * DKP);
            float values[C];
#pragma unroll
            for (int c = 0; c < C; ++c) values[c] = v_of(stage)[tt * kScanCols + C * column_group + c];
            float key[R], dots[C];
#pragma unroll
            for (int c = 0; c < C; ++c) dots[c] = 0.0f;
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 decay4 = g4[(i >> 2) * SPLIT + part], key4 = k4[(i >> 2) * SPLIT + part];
                const float decay[4] = {decay4.x, decay4.y, decay4.z, decay4.w};
                key[i] = key4.x, key[i + 1] = key4.y, key[i + 2] = key4.z, key[i + 3] = key4.w;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        S[c][i + e] *= decay[e];
                        if constexpr (DELTA) dots[c] += S[c][i + e] * key[i + e];
                    }
                }
            }
            if constexpr (DELTA) {
#pragma unroll
                for (int offset = 1; offset < SPLIT; offset <<= 1) {
#pragma unroll
                    for (int c = 0; c < C; ++c) dots[c] += __shfl_xor_sync(0xffffffffu, dots[c], offset);
                }
            }
            float u[C], reads[C];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                u[c] = DELTA ? beta_s[tt] * (values[c] - dots[c]) : values[c];
                reads[c] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 query4 = q4[(i >> 2) * SPLIT + part];
                const float query[4] = {query4.x, query4.y, query4.z, query4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        S[c][i + e] += key[i + e] * u[c];
                        reads[c] += S[c][i + e] * query[e];
                    }
                }
            }
#pragma unroll
            for (int offset = 1; offset < SPLIT; offset <<= 1) {
#pragma unroll
                for (int c = 0; c < C; ++c) reads[c] += __shfl_xor_sync(0xffffffffu, reads[c], offset);
            }
            if (part == 0) {
                float* destination = out + (static_cast<size_t>(start + t0 + tt) * heads + head) * dv + column;
#pragma unroll
                for (int c = 0; c < C; ++c)
                    if (column + c < dv) destination[c] = reads[c];
            }
        }
        __syncthreads();   // this stage is refilled in the next turn
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = ((i >> 2) * SPLIT + part) * 4 + (i & 3);
#pragma unroll
        for (int c = 0; c < C; ++c)
            if (row < dk && column + c < dv) S_base[static_cast<size_t>(row) * dv + column + c] = S[c][i];
    }
}

// grid (tokens, slices of the heads), a warp per head: out[t, h, :] = T(o / sqrt(mean(o^2) + eps) * w * sigmoid(gate[t, h, :])).
template <typename T>
__global__ void gdr_output_kernel(const float* __restrict__ o, const T* __restrict__ ag, int ag_width, int gate_offset,
                                  const float* __restrict__ norm_weight, T* __restrict__ out, int heads, int dv, float eps, int gate_silu) {
    allow_next_kernel();   // the out-projection, launched to start early, may ask for its weights meanwhile
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int head = blockIdx.y * warps + warp; head < heads; head += gridDim.y * warps) {
        const float* row = o + (static_cast<size_t>(token) * heads + head) * dv;
        const T* gate = ag + static_cast<size_t>(token) * ag_width + gate_offset + static_cast<size_t>(head) * dv;
        float sum = 0.0f;
        for (int c = lane; c < dv; c += 32) sum += row[c] * row[c];
        sum = warp_sum(sum);
        const float inv = rsqrtf(sum / static_cast<float>(dv) + eps);
        T* dst = out + (static_cast<size_t>(token) * heads + head) * dv;
        for (int c = lane; c < dv; c += 32) {
            const float z = to_float(gate[c]);
            dst[c] = from_float<T>(row[c] * inv * norm_weight[c] * (gate_silu ? z * sigmoidf_(z) : sigmoidf_(z)));
        }
    }
}

// ------------------------------------------------------------------------------------ long portions in chunks
// The recurrence is linear in the state: S_t = M_t S_{t-1} + k_t (beta_t v_t)^T with M_t = (I - beta_t k_t k_t^T) diag(g_t).
// A long portion is cut into chunks that the scan above runs side by side, each from a zero state and, in dk further
// columns that start as the identity and take zeros as values, the chunk's transition P_t = M_t ... M_1; the scan's
// read-out of those columns is P_t^T q_t.  With S_in the state at a chunk's start,
//   S_t = S0_t + P_t S_in    and    o_t = o0_t + (P_t^T q_t)^T S_in,
// so one short pass over a portion's chunks in order gives every chunk's S_in (and the portion's last state), and one
// pass over the tokens adds the second term to the read-outs.  All in 32-bit.

// state[chunk, head] (dk x (dv + dk)) = [0 | I].  One block per (chunk, head).
__global__ void gdr_chunk_init_kernel(float* __restrict__ chunk_state, int dk, int dv) {
    const int width = dv + dk;
    float* S = chunk_state + static_cast<size_t>(blockIdx.x) * dk * width;
    for (int index = threadIdx.x; index < dk * width; index += blockDim.x) {
        const int row = index / width, col = index - row * width;
        S[index] = col == dv + row ? 1.0f : 0.0f;
    }
}

// grid (long portions, heads, ceil(dv / 32)), block (32, 32): thread (j, y) holds the rows y, y + 32, ... of column j of
// S_in.  long_table rows: (portion, first chunk, chunks).  For each chunk in order: S_in is written to chunk_in[chunk]
// (dk x dv per head), then S_in <- S0_L + P_L S_in, with P_L staged in shared memory where it fits (p_in_shared).  The
// last S_in goes to the portion's state slot, from which the first was read.
constexpr int kPropagateRows = 8;   // dk <= 256
__global__ void __launch_bounds__(1024)
gdr_chunk_propagate_kernel(const float* __restrict__ chunk_state, float* __restrict__ chunk_in, float* __restrict__ state,
                           const int* __restrict__ long_table, const int* __restrict__ segment_slot, int heads, int dk, int dv, int num_slots,
                           int p_in_shared) {
    extern __shared__ float propagate_memory[];
    float* s_in = propagate_memory;          // dk x 32
    float* p_s = propagate_memory + dk * 32;   // dk x (dk + 1) if p_in_shared
    const int portion = long_table[3 * blockIdx.x], first_chunk = long_table[3 * blockIdx.x + 1], chunks = long_table[3 * blockIdx.x + 2];
    const int head = blockIdx.y, j = threadIdx.x, column = blockIdx.z * 32 + j, y = threadIdx.y;
    const int slot = segment_slot[portion];
    if (slot < 0 || slot >= num_slots) return;   // reported by the kernels before
    const bool live = column < dv;
    const int width = dv + dk, pitch = dk + 1;
    float* S_slot = state + (static_cast<size_t>(slot) * heads + head) * dk * dv;
    float mine[kPropagateRows];
#pragma unroll
    for (int r = 0; r < kPropagateRows; ++r) {
        const int row = y + 32 * r;
        mine[r] = (live && row < dk) ? S_slot[static_cast<size_t>(row) * dv + column] : 0.0f;
    }
    for (int c = 0; c < chunks; ++c) {
        const size_t chunk_head = static_cast<size_t>(first_chunk + c) * heads + head;
        float* in_tile = chunk_in + chunk_head * dk * dv;
        const float* S_end = chunk_state + chunk_head * dk * width;   // [S0_L | P_L]
        __syncthreads();   // the turn before has read s_in and p_s
#pragma unroll
        for (int r = 0; r < kPropagateRows; ++r) {
            const int row = y + 32 * r;
            if (row < dk) {
                s_in[row * 32 + j] = mine[r];
                if (live) in_tile[static_cast<size_t>(row) * dv + column] = mine[r];
            }
        }
        if (p_in_shared) {
            for (int index = y * 32 + j; index < dk * dk; index += 1024) {
                const int row = index / dk, m = index - row * dk;
                p_s[row * pitch + m] = S_end[static_cast<size_t>(row) * width + dv + m];
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kPropagateRows; ++r) {
            const int row = y + 32 * r;
            if (row < dk) {
                const float* p_row = p_in_shared ? p_s + row * pitch : S_end + static_cast<size_t>(row) * width + dv;
                float sums[4] = {live ? S_end[static_cast<size_t>(row) * width + column] : 0.0f, 0.0f, 0.0f, 0.0f};
                int m = 0;
                for (; m + 4 <= dk; m += 4) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) sums[e] += p_row[m + e] * s_in[(m + e) * 32 + j];
                }
                for (; m < dk; ++m) sums[0] += p_row[m] * s_in[m * 32 + j];
                mine[r] = (sums[0] + sums[1]) + (sums[2] + sums[3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kPropagateRows; ++r) {
        const int row = y + 32 * r;
        if (live && row < dk) S_slot[static_cast<size_t>(row) * dv + column] = mine[r];
    }
}

// grid (chunks x tiles of 16 tokens, heads): out[t, h, j] = wide[t, h, j] + sum_m wide[t, h, dv + m] * chunk_in[chunk, h, m, j]
// for the tile's tokens, which share what is read of chunk_in.
constexpr int kReadoutTokens = 16;
__global__ void gdr_chunk_readout_kernel(const float* __restrict__ wide, const float* __restrict__ chunk_in, const int* __restrict__ chunk_start,
                                         const int* __restrict__ chunk_length, int tiles_per_chunk, float* __restrict__ out, int heads, int dk, int dv) {
    extern __shared__ __align__(16) float r_s[];   // dk x 16: the tokens' values of one m side by side (zeros past the tile's end)
    const int chunk = blockIdx.x / tiles_per_chunk, tile = blockIdx.x - chunk * tiles_per_chunk, head = blockIdx.y;
    const int first = kReadoutTokens * tile, count = min(kReadoutTokens, chunk_length[chunk] - first);
    if (count <= 0) return;
    const int token0 = chunk_start[chunk] + first;
    for (int index = threadIdx.x; index < kReadoutTokens * dk; index += blockDim.x) {
        const int tt = index / dk, m = index - tt * dk;
        r_s[m * kReadoutTokens + tt] = tt < count ? wide[(static_cast<size_t>(token0 + tt) * heads + head) * (dv + dk) + dv + m] : 0.0f;
    }
    __syncthreads();
    const float* S_in = chunk_in + (static_cast<size_t>(chunk) * heads + head) * dk * dv;
    for (int j = threadIdx.x; j < dv; j += blockDim.x) {
        float sums[kReadoutTokens];
#pragma unroll
        for (int tt = 0; tt < kReadoutTokens; ++tt) sums[tt] = tt < count ? wide[(static_cast<size_t>(token0 + tt) * heads + head) * (dv + dk) + j] : 0.0f;
#pragma unroll 4
        for (int m = 0; m < dk; ++m) {   // four loads of S_in on their way at a time
            const float s = S_in[static_cast<size_t>(m) * dv + j];
            const float4* r4 = reinterpret_cast<const float4*>(r_s + m * kReadoutTokens);
#pragma unroll
            for (int quad = 0; quad < kReadoutTokens / 4; ++quad) {
                const float4 r = r4[quad];
                sums[4 * quad] += r.x * s;
                sums[4 * quad + 1] += r.y * s;
                sums[4 * quad + 2] += r.z * s;
                sums[4 * quad + 3] += r.w * s;
            }
        }
#pragma unroll
        for (int tt = 0; tt < kReadoutTokens; ++tt)
            if (tt < count) out[(static_cast<size_t>(token0 + tt) * heads + head) * dv + j] = sums[tt];
    }
}

template <int DKP, int SPLIT>
inline void launch_scan(dim3 grid, cudaStream_t stream, const float* q, const float* k, const float* g, const float* v, const float* beta,
                        float* state, float* out, const int* segment_start, const int* segment_length, const int* segment_slot, int heads,
                        int groups, int dk, int dv, int num_slots, int* status, const int* segment_list, int v_columns) {
    if (beta != nullptr) {
        static OncePerDevice once;
        allow_shared_memory(once, gdr_scan_kernel<DKP, SPLIT, true>, static_cast<int>(ScanShared<DKP>::kBytes));
        gdr_scan_kernel<DKP, SPLIT, true><<<grid, (kScanCols / kScanThreadCols) * SPLIT, ScanShared<DKP>::kBytes, stream>>>(
            q, k, g, v, beta, state, out, segment_start, segment_length, segment_slot, heads, groups, dk, dv, num_slots, status, segment_list, v_columns);
    } else {
        static OncePerDevice once;
        allow_shared_memory(once, gdr_scan_kernel<DKP, SPLIT, false>, static_cast<int>(ScanShared<DKP>::kBytes));
        gdr_scan_kernel<DKP, SPLIT, false><<<grid, (kScanCols / kScanThreadCols) * SPLIT, ScanShared<DKP>::kBytes, stream>>>(
            q, k, g, v, beta, state, out, segment_start, segment_length, segment_slot, heads, groups, dk, dv, num_slots, status, segment_list, v_columns);
    }
}

}  // namespace lb

extern "C" {

int lb_gdr_prepare(const void* proj, int proj_width, const void* ag, int ag_width, void* conv_state, const float* conv_weight,
                   const float* a_log, const float* dt_bias, float* q_out, float* k_out, float* v_out, float* beta_out, float* g_out,
                   const int* token_segment, const int* segment_start, const int* segment_slot, int tokens, int heads, int groups, int dk,
                   int dv, int taps, int num_slots, float unit_eps, float q_scale, int dtype, int* status, cudaStream_t stream, int update_state,
                   int decay_per_head) {
    if (tokens == 0) return 0;
    if (dk > 32 * lb::kPrepareMaxPerLane || taps < 1 || heads % groups != 0) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        const int units = 2 * groups + 2 * heads;
        const dim3 grid(tokens, (units + 3) / 4);
        if (update_state)
            lb::gdr_prepare_kernel<T, true><<<grid, 128, 0, stream>>>(static_cast<const T*>(proj), proj_width, static_cast<const T*>(ag), ag_width,
                                                                       static_cast<T*>(conv_state), conv_weight, a_log, dt_bias, q_out, k_out, v_out, beta_out, g_out,
                                                                       token_segment, segment_start, segment_slot, heads, groups, dk, dv, taps, num_slots, unit_eps,
                                                                       q_scale, status, decay_per_head);
        else
            lb::gdr_prepare_kernel<T, false><<<grid, 128, 0, stream>>>(static_cast<const T*>(proj), proj_width, static_cast<const T*>(ag), ag_width,
                                                                        static_cast<const T*>(conv_state), conv_weight, a_log, dt_bias, q_out, k_out, v_out, beta_out,
                                                                        g_out, token_segment, segment_start, segment_slot, heads, groups, dk, dv, taps, num_slots,
                                                                        unit_eps, q_scale, status, decay_per_head);
    })
    return LB_LAUNCH_RESULT();
}

int lb_gdr_conv_state(const void* proj, int proj_width, void* conv_state, const int* segment_start, const int* segment_length,
                      const int* segment_slot, int segments, int channels, int taps, int num_slots, int dtype, cudaStream_t stream) {
    if (segments == 0 || taps <= 1) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::gdr_conv_state_kernel<T><<<dim3(segments, (channels + 255) / 256), 256, 0, stream>>>(static_cast<const T*>(proj), proj_width, static_cast<T*>(conv_state), segment_start,
                                                                   segment_length, segment_slot, channels, taps, num_slots);
    })
    return LB_LAUNCH_RESULT();
}

// segment_list (may be null): the portions to run, `segments` of them.  v_columns: the columns `v` has (0: dv).
// beta null: the plain linear recurrence (no delta rule).
int lb_gdr_scan(const float* q, const float* k, const float* g, const float* v, const float* beta, float* state, float* out,
                const int* segment_start, const int* segment_length, const int* segment_slot, int segments, int heads, int groups, int dk, int dv,
                int num_slots, int* status, cudaStream_t stream, const int* segment_list, int v_columns) {
    if (segments == 0) return 0;
    if (v_columns <= 0) v_columns = dv;
    if (dk < 1 || dk > 256 || dv < 1 || heads % groups != 0 || v_columns > dv) return -2;
    const dim3 grid(segments, heads, (dv + lb::kScanCols - 1) / lb::kScanCols);
    if (dk <= 32)
        lb::launch_scan<32, 4>(grid, stream, q, k, g, v, beta, state, out, segment_start, segment_length, segment_slot, heads, groups, dk, dv, num_slots, status, segment_list, v_columns);
    else if (dk <= 64)
        lb::launch_scan<64, 8>(grid, stream, q, k, g, v, beta, state, out, segment_start, segment_length, segment_slot, heads, groups, dk, dv, num_slots, status, segment_list, v_columns);
    else if (dk <= 128)
        lb::launch_scan<128, 16>(grid, stream, q, k, g, v, beta, state, out, segment_start, segment_length, segment_slot, heads, groups, dk, dv, num_slots, status, segment_list, v_columns);
    else
        lb::launch_scan<256, 32>(grid, stream, q, k, g, v, beta, state, out, segment_start, segment_length, segment_slot, heads, groups, dk, dv, num_slots, status, segment_list, v_columns);
    return LB_LAUNCH_RESULT();
}

// The passes around the chunks' scan (which is lb_gdr_scan over the chunk tables with dv + dk columns): `chunk_state`
// [chunks, heads, dk, dv + dk] is set to [0 | I] by lb_gdr_chunk_init before the scan; after it lb_gdr_chunk_finish gives every
// chunk its incoming state (`chunk_in` [chunks, heads, dk, dv]), the portions' slots their last state, and the tokens
// of chunks their read-out (`wide` [tokens, heads, dv + dk] is what the scan wrote; `out` [tokens, heads, dv]).
int lb_gdr_chunk_init(float* chunk_state, int chunks, int heads, int dk, int dv, cudaStream_t stream) {
    if (chunks == 0) return 0;
    lb::gdr_chunk_init_kernel<<<chunks * heads, 256, 0, stream>>>(chunk_state, dk, dv);
    return LB_LAUNCH_RESULT();
}

int lb_gdr_chunk_finish(const float* chunk_state, float* chunk_in, float* state, const float* wide, float* out, const int* long_table, int long_portions,
                        const int* segment_slot, const int* chunk_start, const int* chunk_length, int chunks, int chunk_tokens, int heads, int dk, int dv,
                        int num_slots, cudaStream_t stream) {
    if (long_portions == 0 || chunks == 0) return 0;
    if (dk > 32 * lb::kPropagateRows || chunk_tokens < 1) return -2;
    size_t shared = static_cast<size_t>(dk) * 32 * sizeof(float);
    const size_t with_p = shared + static_cast<size_t>(dk) * (dk + 1) * sizeof(float);
    const int p_in_shared = with_p <= 160 * 1024 ? 1 : 0;
    if (p_in_shared) shared = with_p;
    static lb::OncePerDevice once;
    lb::allow_shared_memory(once, lb::gdr_chunk_propagate_kernel, 160 * 1024);
    lb::gdr_chunk_propagate_kernel<<<dim3(long_portions, heads, (dv + 31) / 32), dim3(32, 32), shared, stream>>>(
        chunk_state, chunk_in, state, long_table, segment_slot, heads, dk, dv, num_slots, p_in_shared);
    const int tiles_per_chunk = (chunk_tokens + lb::kReadoutTokens - 1) / lb::kReadoutTokens;
    lb::gdr_chunk_readout_kernel<<<dim3(chunks * tiles_per_chunk, heads), 128, static_cast<size_t>(lb::kReadoutTokens) * dk * sizeof(float), stream>>>(
        wide, chunk_in, chunk_start, chunk_length, tiles_per_chunk, out, heads, dk, dv);
    return LB_LAUNCH_RESULT();
}

int lb_gdr_output(const float* o, const void* ag, int ag_width, int gate_offset, const float* norm_weight, void* out, int tokens, int heads, int dv,
                  float eps, int dtype, cudaStream_t stream, int gate_silu) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::gdr_output_kernel<T><<<dim3(tokens, (heads + 3) / 4), 128, 0, stream>>>(o, static_cast<const T*>(ag), ag_width, gate_offset, norm_weight, static_cast<T*>(out), heads, dv, eps, gate_silu);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
