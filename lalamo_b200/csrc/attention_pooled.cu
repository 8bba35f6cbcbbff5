// Sigmoid-weighted attention under a sliding window with pooled blocks before it.
//
// A token at position i sees the keys j with 0 <= i - j < window and, beside them, one mean key and one mean value
// for every block of `pool` consecutive positions that lies wholly before the window: block b covers b pool ..
// b pool + pool - 1 and is seen if b pool + pool - 1 <= i - window.  Positions that have left the window and whose
// block is not yet whole behind it are not seen.  A visible key (token or block alike) weighs
//   w = sigmoid(cap * tanh(q . k * scale / cap) + bias[head])      (cap <= 0: no cap)
// and the output is the plain sum of w times the value: no softmax, no denominator.  Values may be rotated by their
// position before they are cached (all their channels, pair m turning by j * freq[m]); the head's sum is then turned
// back by the query's position, so that a value acts through the distance i - j.
//
// Four kernels: `pooled_rewrite` (rotation of q, k and v in 32-bit, one rounding, pages written), `pooled_means` (the mean
// of every block that the step completes, from the pages, into the pooled pages), `pooled_attention_plain` (a block per token
// and head, everything 32-bit: the 32-bit path and the reference for the tensor-core kernel) and `pooled_attention_mma`
// (bfloat16 on mma.sync m16n8k16: a CTA takes 16 consecutive tokens of a portion and the query heads of one K/V head).
// Keys are summed in the order blocks 0, 1, ... then positions upwards, whatever the step's cutting.
//
// Token pages: keys [page][row][group][dk], values transposed [page][group][dv][row], `page_size` rows a page, found
// through the token block table (block = position / page_size).  Pooled pages: the same with `pool_rows` rows a page,
// block b in page pool_table[b / pool_rows], row b % pool_rows.
#include "common.cuh"

namespace lb {

struct PooledLayout {
    int page_size, num_pages, max_blocks;             // token pages and their block table
    int pool_rows, pool_pages, pool_max_blocks;       // pooled pages and theirs
    int groups, dk, dv;
};

__device__ __forceinline__ int token_page(const int* __restrict__ table, const PooledLayout& L, int segment, int position) {
    const int block = position / L.page_size;
    if (block >= L.max_blocks) return -1;
    const int page = table[static_cast<size_t>(segment) * L.max_blocks + block];
    return page >= 0 && page < L.num_pages ? page : -1;
}

__device__ __forceinline__ int pooled_page(const int* __restrict__ table, const PooledLayout& L, int segment, int block_index) {
    const int block = block_index / L.pool_rows;
    if (block >= L.pool_max_blocks) return -1;
    const int page = table[static_cast<size_t>(segment) * L.pool_max_blocks + block];
    return page >= 0 && page < L.pool_pages ? page : -1;
}

// The pair partner and the sign of a rotation in halves (m with m + dims / 2) or of neighbours (2m with 2m + 1):
// channel c of the first `dims` turns to x[c] cos a + sign x[partner] sin a with a = position * freq[pair].
__device__ __forceinline__ void rotation_pair(int c, int dims, int interleaved, int& partner, int& pair, float& sign) {
    if (interleaved) {
        pair = c >> 1;
        partner = c ^ 1;
        sign = (c & 1) ? 1.0f : -1.0f;
    } else {
        const int half = dims >> 1;
        pair = c < half ? c : c - half;
        partner = c < half ? c + half : c - half;
        sign = c < half ? -1.0f : 1.0f;
    }
}

// grid (tokens): q [tokens, heads, dk] rotated into q_out; k rotated and v (rotated over all dv channels if v_freq is
// given) into the token's page row.  qkv rows: q (heads x dk) | k (groups x dk) | v (groups x dv), row stride `stride`.
template <typename T>
__global__ void pooled_rewrite_kernel(const T* __restrict__ qkv, int stride, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                      const float* __restrict__ qk_freq, int rot_dims, int qk_interleaved, const float* __restrict__ v_freq,
                                      int v_interleaved, const int* __restrict__ positions, const int* __restrict__ token_segment,
                                      const int* __restrict__ block_table, PooledLayout L, int heads, int write_kv, int* status) {
    const int token = blockIdx.x;
    const int position = positions[token];
    const int segment = token_segment[token];
    const T* row = qkv + static_cast<size_t>(token) * stride;
    const int q_width = heads * L.dk, k_width = L.groups * L.dk, v_width = L.groups * L.dv;
    const float p = static_cast<float>(position);
    for (int index = threadIdx.x; index < q_width + k_width; index += blockDim.x) {
        const int c = index % L.dk;
        float value = to_float(row[index]);
        if (c < rot_dims) {
            int partner, pair;
            float sign;
            rotation_pair(c, rot_dims, qk_interleaved, partner, pair, sign);
            float sine, cosine;
            sincosf(p * qk_freq[pair], &sine, &cosine);
            value = value * cosine + sign * to_float(row[index - c + partner]) * sine;
        }
        if (index < q_width) {
            q_out[static_cast<size_t>(token) * q_width + index] = from_float<T>(value);
        } else if (write_kv) {
            const int page = token_page(block_table, L, segment, position);
            if (page < 0) {
                report_error(status, kBadPage);
                continue;
            }
            const int kc = index - q_width;   // group * dk + c
            k_pages[(static_cast<size_t>(page) * L.page_size + position % L.page_size) * k_width + kc] = from_float<T>(value);
        }
    }
    if (!write_kv) return;
    const int page = token_page(block_table, L, segment, position);
    if (page < 0) return;   // reported above
    for (int index = threadIdx.x; index < v_width; index += blockDim.x) {
        const int c = index % L.dv;
        float value = to_float(row[q_width + k_width + index]);
        if (v_freq != nullptr) {
            int partner, pair;
            float sign;
            rotation_pair(c, L.dv, v_interleaved, partner, pair, sign);
            float sine, cosine;
            sincosf(p * v_freq[pair], &sine, &cosine);
            value = value * cosine + sign * to_float(row[q_width + k_width + index - c + partner]) * sine;
        }
        // values transposed: [page][group][channel][row]
        v_pages[(static_cast<size_t>(page) * v_width + index) * L.page_size + position % L.page_size] = from_float<T>(value);
    }
}

// grid (portions, blocks a portion can complete): block `first + blockIdx.y` of the request, if this step wrote its last
// position, gets the mean of its `pool` keys and values as the pages hold them (sums in 32-bit in the order of the
// positions, divided by pool, rounded once).
template <typename T>
__global__ void pooled_means_kernel(const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ pk_pages, T* __restrict__ pv_pages,
                                    const int* __restrict__ segment_length, const int* __restrict__ segment_context,
                                    const int* __restrict__ block_table, const int* __restrict__ pool_table, PooledLayout L, int pool, int* status) {
    const int segment = blockIdx.x;
    const int context = segment_context[segment], length = segment_length[segment];
    // blocks whose last position lies in [context, context + length)
    const int first = context / pool;
    const int block_index = first + blockIdx.y;
    const int last_position = block_index * pool + pool - 1;
    if (last_position >= context + length) return;
    const int out_page = pooled_page(pool_table, L, segment, block_index);
    if (out_page < 0) {
        if (threadIdx.x == 0) report_error(status, kBadPage);
        return;
    }
    const int out_row = block_index % L.pool_rows;
    const int k_width = L.groups * L.dk, v_width = L.groups * L.dv;
    const float inverse = 1.0f / static_cast<float>(pool);
    for (int index = threadIdx.x; index < k_width + v_width; index += blockDim.x) {
        float sum = 0.0f;
        bool bad = false;
        for (int j = 0; j < pool; ++j) {
            const int position = block_index * pool + j;
            const int page = token_page(block_table, L, segment, position);
            if (page < 0) {
                bad = true;
                break;
            }
            const int r = position % L.page_size;
            sum += index < k_width ? to_float(k_pages[(static_cast<size_t>(page) * L.page_size + r) * k_width + index])
                                   : to_float(v_pages[(static_cast<size_t>(page) * v_width + (index - k_width)) * L.page_size + r]);
        }
        if (bad) {
            report_error(status, kBadPage);
            continue;
        }
        if (index < k_width)
            pk_pages[(static_cast<size_t>(out_page) * L.pool_rows + out_row) * k_width + index] = from_float<T>(sum * inverse);
        else
            pv_pages[(static_cast<size_t>(out_page) * v_width + (index - k_width)) * L.pool_rows + out_row] = from_float<T>(sum * inverse);
    }
}

__device__ __forceinline__ float pooled_weight(float dot, float scale, float cap, float bias) {
    float s = dot * scale;
    if (cap > 0.0f) s = cap * tanhf(s / cap);
    return 1.0f / (1.0f + expf(-(s + bias)));
}

constexpr int kPooledChunk = 128, kPooledThreads = 128, kPooledMaxDims = 4;   // dv <= 512

// grid (tokens, heads).  Items: the visible blocks 0 .. blocks - 1, then the positions first .. i; 128 at a time, a
// thread per item for the weights, a thread per channel for the sums (in item order).
template <typename T>
__global__ void __launch_bounds__(kPooledThreads)
pooled_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages, const T* __restrict__ pk_pages,
                              const T* __restrict__ pv_pages, T* __restrict__ out, const int* __restrict__ positions,
                              const int* __restrict__ token_segment, const int* __restrict__ block_table, const int* __restrict__ pool_table,
                              PooledLayout L, int heads, float scale, float cap, const float* __restrict__ head_bias, int window, int pool,
                              const float* __restrict__ v_freq, int v_interleaved, int* status) {
    extern __shared__ float shared[];
    float* q_s = shared;                 // dk
    float* weights = q_s + L.dk;         // kPooledChunk
    int* rows = reinterpret_cast<int*>(weights + kPooledChunk);   // kPooledChunk: page * rows-per-page + row, or -1
    float* turned = reinterpret_cast<float*>(rows + kPooledChunk);   // dv
    const int token = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int group = head / (heads / L.groups);
    const int segment = token_segment[token], position = positions[token];
    const int first = max(0, position - window + 1);
    const int blocks = pool > 0 ? max(0, position - window + 1) / pool : 0;
    const float bias = head_bias != nullptr ? head_bias[head] : 0.0f;
    for (int d = tid; d < L.dk; d += blockDim.x) q_s[d] = to_float(q[(static_cast<size_t>(token) * heads + head) * L.dk + d]);
    __syncthreads();
    float acc[kPooledMaxDims];
#pragma unroll
    for (int slot = 0; slot < kPooledMaxDims; ++slot) acc[slot] = 0.0f;
    const int k_width = L.groups * L.dk, v_width = L.groups * L.dv;
    const int items = blocks + (position + 1 - first);
    for (int chunk = 0; chunk < items; chunk += kPooledChunk) {
        const int count = min(kPooledChunk, items - chunk);
        if (tid < count) {
            const int item = chunk + tid;
            const bool pooled = item < blocks;
            const int where = pooled ? item : first + (item - blocks);
            const int page = pooled ? pooled_page(pool_table, L, segment, where) : token_page(block_table, L, segment, where);
            float w = 0.0f;
            int row_index = -1;
            if (page < 0) {
                report_error(status, kBadPage);
            } else {
                const int per_page = pooled ? L.pool_rows : L.page_size;
                row_index = page * per_page + where % per_page;
                const T* k_row = (pooled ? pk_pages : k_pages) + static_cast<size_t>(row_index) * k_width + group * L.dk;
                float dot = 0.0f;
                for (int d = 0; d < L.dk; ++d) dot += q_s[d] * to_float(k_row[d]);
                w = pooled_weight(dot, scale, cap, bias);
            }
            weights[tid] = w;
            rows[tid] = row_index;
        }
        __syncthreads();
#pragma unroll
        for (int slot = 0; slot < kPooledMaxDims; ++slot) {
            const int d = tid + slot * kPooledThreads;
            if (d < L.dv) {
                float sum = acc[slot];
                for (int i = 0; i < count; ++i) {
                    const int row_index = rows[i];
                    if (row_index < 0) continue;
                    const bool pooled = chunk + i < blocks;
                    const int per_page = pooled ? L.pool_rows : L.page_size;
                    const int page = row_index / per_page, r = row_index - page * per_page;
                    const T* base = pooled ? pv_pages : v_pages;
                    sum += weights[i] * to_float(base[(static_cast<size_t>(page) * v_width + group * L.dv + d) * per_page + r]);
                }
                acc[slot] = sum;
            }
        }
        __syncthreads();
    }
    T* dst = out + (static_cast<size_t>(token) * heads + head) * L.dv;
    if (v_freq == nullptr) {
#pragma unroll
        for (int slot = 0; slot < kPooledMaxDims; ++slot) {
            const int d = tid + slot * kPooledThreads;
            if (d < L.dv) dst[d] = from_float<T>(acc[slot]);
        }
        return;
    }
#pragma unroll
    for (int slot = 0; slot < kPooledMaxDims; ++slot) {
        const int d = tid + slot * kPooledThreads;
        if (d < L.dv) turned[d] = acc[slot];
    }
    __syncthreads();
    const float p = static_cast<float>(position);
#pragma unroll
    for (int slot = 0; slot < kPooledMaxDims; ++slot) {
        const int d = tid + slot * kPooledThreads;
        if (d < L.dv) {
            int partner, pair;
            float sign;
            rotation_pair(d, L.dv, v_interleaved, partner, pair, sign);
            float sine, cosine;
            sincosf(p * v_freq[pair], &sine, &cosine);
            dst[d] = from_float<T>(turned[d] * cosine - sign * turned[partner] * sine);   // the turn by -position
        }
    }
}

}  // namespace lb

extern "C" {

int lb_pooled_rewrite(const void* qkv, int stride, void* q_out, void* k_pages, void* v_pages, const float* qk_freq, int rot_dims, int qk_interleaved,
                      const float* v_freq, int v_interleaved, const int* positions, const int* token_segment, const int* block_table, int tokens,
                      int heads, int groups, int dk, int dv, int page_size, int num_pages, int max_blocks, int write_kv, int dtype, int* status,
                      cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (heads % groups != 0 || rot_dims < 0 || rot_dims > dk || rot_dims % 2 != 0 || (v_freq != nullptr && dv % 2 != 0)) return -2;
    lb::PooledLayout L{page_size, num_pages, max_blocks, 1, 0, 0, groups, dk, dv};
    LB_DISPATCH_DTYPE(dtype, {
        lb::pooled_rewrite_kernel<T><<<tokens, 256, 0, stream>>>(static_cast<const T*>(qkv), stride, static_cast<T*>(q_out), static_cast<T*>(k_pages),
                                                                  static_cast<T*>(v_pages), qk_freq, rot_dims, qk_interleaved, v_freq, v_interleaved, positions,
                                                                  token_segment, block_table, L, heads, write_kv, status);
    })
    return LB_LAUNCH_RESULT();
}

// max_length: the longest portion of the step (a portion of n tokens completes at most n / pool + 1 blocks).
int lb_pooled_means(const void* k_pages, const void* v_pages, void* pk_pages, void* pv_pages, const int* segment_length, const int* segment_context,
                    const int* block_table, const int* pool_table, int segments, int max_length, int groups, int dk, int dv, int page_size, int num_pages,
                    int max_blocks, int pool_rows, int pool_pages, int pool_max_blocks, int pool, int dtype, int* status, cudaStream_t stream) {
    if (segments == 0 || max_length == 0) return 0;
    if (pool < 1 || pool_rows < 1) return -2;
    lb::PooledLayout L{page_size, num_pages, max_blocks, pool_rows, pool_pages, pool_max_blocks, groups, dk, dv};
    const dim3 grid(segments, max_length / pool + 1);
    LB_DISPATCH_DTYPE(dtype, {
        lb::pooled_means_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(k_pages), static_cast<const T*>(v_pages), static_cast<T*>(pk_pages),
                                                              static_cast<T*>(pv_pages), segment_length, segment_context, block_table, pool_table, L, pool, status);
    })
    return LB_LAUNCH_RESULT();
}

int lb_pooled_attention_plain(const void* q, const void* k_pages, const void* v_pages, const void* pk_pages, const void* pv_pages, void* out,
                              const int* positions, const int* token_segment, const int* block_table, const int* pool_table, int tokens, int heads,
                              int groups, int dk, int dv, int page_size, int num_pages, int max_blocks, int pool_rows, int pool_pages, int pool_max_blocks,
                              float scale, float cap, const float* head_bias, int window, int pool, const float* v_freq, int v_interleaved, int dtype,
                              int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (heads % groups != 0 || dv > lb::kPooledThreads * lb::kPooledMaxDims || window < 1 || pool < 0) return -2;
    lb::PooledLayout L{page_size, num_pages, max_blocks, pool_rows > 0 ? pool_rows : 1, pool_pages, pool_max_blocks, groups, dk, dv};
    const size_t shared = (static_cast<size_t>(dk) + 2 * lb::kPooledChunk + dv) * sizeof(float);
    if (shared > 48 * 1024) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        lb::pooled_attention_plain_kernel<T><<<dim3(tokens, heads), lb::kPooledThreads, shared, stream>>>(
            static_cast<const T*>(q), static_cast<const T*>(k_pages), static_cast<const T*>(v_pages), static_cast<const T*>(pk_pages),
            static_cast<const T*>(pv_pages), static_cast<T*>(out), positions, token_segment, block_table, pool_table, L, heads, scale, cap, head_bias, window,
            pool, v_freq, v_interleaved, status);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
