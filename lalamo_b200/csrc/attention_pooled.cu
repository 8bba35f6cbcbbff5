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
// (bfloat16 on mma.sync m16n8k16: a CTA takes up to 64 consecutive tokens of a portion and up to four query heads of one K/V head).
// Keys are summed in the order blocks 0, 1, ... then positions upwards, whatever the step's cutting.
//
// Pages: a row holds all a position leaves behind, [page][row][group][key (dk) | value (dv)], `page_size` rows a page, found
// through the token block table (block = position / page_size).  Pooled pages: the same with `pool_rows` rows a page,
// block b in page pool_table[b / pool_rows], row b % pool_rows.
#include "common.cuh"

#include <type_traits>

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
__global__ void pooled_rewrite_kernel(const T* __restrict__ qkv, int stride, T* __restrict__ q_out, T* __restrict__ pages,
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
            const int group = (index - q_width) / L.dk;
            pages[((static_cast<size_t>(page) * L.page_size + position % L.page_size) * L.groups + group) * (L.dk + L.dv) + c] = from_float<T>(value);
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
        pages[((static_cast<size_t>(page) * L.page_size + position % L.page_size) * L.groups + index / L.dv) * (L.dk + L.dv) + L.dk + c] = from_float<T>(value);
    }
}

// grid (portions, blocks a portion can complete): block `first + blockIdx.y` of the request, if this step wrote its last
// position, gets the mean of its `pool` keys and values as the pages hold them (sums in 32-bit in the order of the
// positions, divided by pool, rounded once).
template <typename T>
__global__ void pooled_means_kernel(const T* __restrict__ pages, T* __restrict__ pooled_pages,
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
    const int width = L.groups * (L.dk + L.dv);   // a row: every group's key and value
    const float inverse = 1.0f / static_cast<float>(pool);
    for (int index = threadIdx.x; index < width; index += blockDim.x) {
        float sum = 0.0f;
        bool bad = false;
        for (int j = 0; j < pool; ++j) {
            const int position = block_index * pool + j;
            const int page = token_page(block_table, L, segment, position);
            if (page < 0) {
                bad = true;
                break;
            }
            sum += to_float(pages[(static_cast<size_t>(page) * L.page_size + position % L.page_size) * width + index]);
        }
        if (bad) {
            report_error(status, kBadPage);
            continue;
        }
        pooled_pages[(static_cast<size_t>(out_page) * L.pool_rows + out_row) * width + index] = from_float<T>(sum * inverse);
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
pooled_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pages, const T* __restrict__ pooled_pages, T* __restrict__ out,
                              const int* __restrict__ positions,
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
    const int width = L.groups * (L.dk + L.dv);
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
                const T* k_row = (pooled ? pooled_pages : pages) + static_cast<size_t>(row_index) * width + group * (L.dk + L.dv);
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
                    const T* base = chunk + i < blocks ? pooled_pages : pages;
                    sum += weights[i] * to_float(base[static_cast<size_t>(row_index) * width + group * (L.dk + L.dv) + L.dk + d]);
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

// ------------------------------------------------------------------------------------ tensor cores (bfloat16)
// A CTA of eight warps takes a tile of up to 16 * TB consecutive tokens of one portion and HB query heads of one K/V head
// (HB * TB = 8, HB at most 4: a warp is one head's 16 tokens).  Rows of the cache come 64 at a time through four cp.async stages, first the
// pooled blocks from block 0 on, then the positions from the multiple of 64 at or below the tile's first visible one: so the
// tiles a query's keys fall into, and with them the order of its sums, depend on its position alone.  Rows that no query
// of the CTA sees are zero-filled and never read.  S = Q K^T (m16n8k16, K through ldmatrix from the rows), the weights in 32-bit with
// a mask per element, P rounded to bfloat16 as the next product's A operand, O += P V with V through ldmatrix.trans from the
// same rows.  At the end a head's sums are turned back by the query's position in registers (both channels of a pair lie in
// one thread) and rounded once.  Where a launch has few CTAs (single decoded tokens), grid.z CTAs share out a tile's blocks of 64
// rows; each writes its 32-bit sums, and `pooled_finish` adds them in the order of the shares, turns them back and rounds.
constexpr int kPooledMmaKeys = 64, kPooledMmaWarps = 8, kPooledMmaStages = 4;   // three tiles on their way while one is worked on

__device__ __forceinline__ void pooled_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void pooled_ldmatrix_x4_trans(uint32_t (&r)[4], const void* shared_address) {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(shared_address));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

__device__ __forceinline__ void pooled_ldmatrix_x4(uint32_t (&r)[4], const void* shared_address) {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(shared_address));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

// 16 bytes from global to shared memory, or 16 zero bytes (nothing is read) if `valid` is false.
__device__ __forceinline__ void pooled_copy_16(void* shared_destination, const void* global_source, bool valid) {
    const uint32_t destination = static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(destination), "l"(global_source), "r"(bytes) : "memory");
}

// The weight of a score in as few instructions as it takes, through the fast base-2 exponential and reciprocal (relative errors
// near 2^-22; the approximate tanh instruction's absolute error of 2^-11, times a cap of tens, would move a score by more than
// bfloat16 rounding does):  tanh(x) = 1 - 2 r with r = 1 / (1 + 2^(2 x log2 e)),  sigmoid(y) = 1 / (1 + 2^(-y log2 e)).
__device__ __forceinline__ float pooled_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float pooled_reciprocal(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
struct PooledWeight {
    float to_exponent, slope, offset;   // capped: e = 2^(s to_exponent), r = 1 / (1 + e), w = 1 / (1 + 2^(r slope + offset)); plain: w = 1 / (1 + 2^(s slope + offset))
    bool capped;
    __device__ __forceinline__ PooledWeight(float scale, float cap, float bias) {
        constexpr float kLog2e = 1.4426950408889634f;
        capped = cap > 0.0f;
        if (capped) {
            // score = cap (1 - 2 r);  -(score + bias) log2 e = r (2 cap log2 e) - (cap + bias) log2 e
            to_exponent = 2.0f * scale / cap * kLog2e;
            slope = 2.0f * cap * kLog2e;
            offset = -(cap + bias) * kLog2e;
        } else {
            to_exponent = 0.0f;
            slope = -scale * kLog2e;
            offset = -bias * kLog2e;
        }
    }
    __device__ __forceinline__ float operator()(float dot) const {
        const float x = capped ? pooled_reciprocal(1.0f + pooled_exp2(dot * to_exponent)) : dot;
        return pooled_reciprocal(1.0f + pooled_exp2(fmaf(x, slope, offset)));
    }
    // the same with the branch decided at compile time, for loops whose elements should interleave
    template <bool CAPPED>
    __device__ __forceinline__ float value(float dot) const {
        const float x = CAPPED ? pooled_reciprocal(1.0f + pooled_exp2(dot * to_exponent)) : dot;
        return pooled_reciprocal(1.0f + pooled_exp2(fmaf(x, slope, offset)));
    }
};

__device__ __forceinline__ uint32_t pooled_pack(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

// tiles: (first row, count) per tile.  grid (tiles, groups * ceil(heads per group / HB)).  DK, DV: the largest key and
// value sizes of the instantiation (multiples of 16); the real ones, multiples of 16 too, come in L.
template <int DK, int DV>
__global__ void __launch_bounds__(32 * kPooledMmaWarps)
pooled_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pages, const __nv_bfloat16* __restrict__ pooled_pages,
                            __nv_bfloat16* __restrict__ out, const int* __restrict__ tiles, const int* __restrict__ positions,
                            const int* __restrict__ token_segment, const int* __restrict__ block_table, const int* __restrict__ pool_table,
                            PooledLayout L, int heads, int head_block, float scale, float cap, const float* __restrict__ head_bias, int window, int pool,
                            const float* __restrict__ v_freq, int v_interleaved, int* status, float* __restrict__ partial, int total_rows) {
    // partial (null if gridDim.z is 1): [share][row][head][dv], 32-bit sums not yet turned back
    extern __shared__ __align__(16) __nv_bfloat16 pooled_rows[];   // kPooledMmaStages stages of 64 rows of `pitch` elements
    const int row_width = L.dk + L.dv, pitch = row_width + 8;      // rows 16 bytes apart modulo 128: no bank is met twice
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int first_row = tiles[2 * blockIdx.x], count = tiles[2 * blockIdx.x + 1];
    const int per_group = heads / L.groups, head_blocks = (per_group + head_block - 1) / head_block;
    const int group = blockIdx.y / head_blocks, head_in_group = (blockIdx.y % head_blocks) * head_block + warp % head_block;
    const int token_block = warp / head_block;                     // the warp's 16 tokens of the tile
    const bool idle = head_in_group >= per_group || token_block * 16 >= count || token_block >= kPooledMmaWarps / head_block;
    const int head = group * per_group + (idle ? 0 : head_in_group);
    const int segment = token_segment[first_row];
    const int p_first = positions[first_row], p_last = p_first + count - 1;   // a tile's tokens follow one another in a portion
    const int blocks_seen = pool > 0 ? max(0, p_last - window + 1) / pool : 0;   // by the tile's last token
    const int first_key = max(0, p_first - window + 1);
    const int pooled_tiles = (blocks_seen + kPooledMmaKeys - 1) / kPooledMmaKeys;
    const int first_token_tile = first_key / kPooledMmaKeys, token_tiles = p_last / kPooledMmaKeys - first_token_tile + 1;
    const int all_tiles = pooled_tiles + token_tiles;
    const int tile_begin = static_cast<int>(static_cast<long long>(all_tiles) * blockIdx.z / gridDim.z);
    const int tile_end = static_cast<int>(static_cast<long long>(all_tiles) * (blockIdx.z + 1) / gridDim.z);
    const int chunks = row_width / 8;   // 16-byte pieces of a row
    const size_t group_offset = static_cast<size_t>(group) * row_width, row_stride = static_cast<size_t>(L.groups) * row_width;

    // Four threads copy a row, 16 bytes each and turn; the row's page is looked up a tile ahead (while the tile before is worked on),
    // so that no copy waits for its block-table entry.
    const int load_row = threadIdx.x >> 2, load_part = threadIdx.x & 3;
    auto lookup = [&](int tile) -> int {   // the page of this thread's row of the tile, -1 if the row is not to be read
        if (tile >= tile_end) return -1;
        const bool pooled = tile < pooled_tiles;
        const int where = (pooled ? tile * kPooledMmaKeys : (first_token_tile + tile - pooled_tiles) * kPooledMmaKeys) + load_row;
        if (!(pooled ? where < blocks_seen : (where >= first_key && where <= p_last))) return -1;
        const int page = pooled ? pooled_page(pool_table, L, segment, where) : token_page(block_table, L, segment, where);
        if (page < 0) report_error(status, kBadPage);
        return page;
    };
    int page_ahead = lookup(tile_begin);
    auto load = [&](int tile) {   // a tile past the CTA's last is an empty group: every turn commits one, so that one wait fits all
        if (tile >= tile_end) {
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            return;
        }
        __nv_bfloat16* destination = pooled_rows + (static_cast<size_t>(tile % kPooledMmaStages) * kPooledMmaKeys + load_row) * pitch;
        const bool pooled = tile < pooled_tiles;
        const int where = (pooled ? tile * kPooledMmaKeys : (first_token_tile + tile - pooled_tiles) * kPooledMmaKeys) + load_row;
        const int page = page_ahead;
        const int per_page = pooled ? L.pool_rows : L.page_size;
        const __nv_bfloat16* source = (pooled ? pooled_pages : pages) + (page < 0 ? 0 : (static_cast<size_t>(page) * per_page + where % per_page) * row_stride + group_offset);
        for (int chunk = load_part; chunk < chunks; chunk += 4) pooled_copy_16(destination + 8 * chunk, source + 8 * chunk, page >= 0);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        page_ahead = lookup(tile + 1);
    };
#pragma unroll
    for (int ahead = 0; ahead < kPooledMmaStages - 1; ++ahead) load(tile_begin + ahead);

    // the warp's queries as A fragments, its rows' positions and what each of them sees
    const int row_g = token_block * 16 + g, row_g8 = row_g + 8;
    const bool live_g = !idle && row_g < count, live_g8 = !idle && row_g8 < count;
    const int p_g = p_first + row_g, p_g8 = p_first + row_g8;
    const int seen_g = pool > 0 ? max(0, p_g - window + 1) / pool : 0, seen_g8 = pool > 0 ? max(0, p_g8 - window + 1) / pool : 0;
    uint32_t q_a[DK / 16][4];
    {
        const __nv_bfloat16* q_g = q + (static_cast<size_t>(first_row + row_g) * heads + head) * L.dk;
        const __nv_bfloat16* q_g8 = q + (static_cast<size_t>(first_row + row_g8) * heads + head) * L.dk;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            const bool in_k = 16 * ks < L.dk;
            q_a[ks][0] = live_g && in_k ? *reinterpret_cast<const uint32_t*>(q_g + 16 * ks + 2 * t) : 0u;
            q_a[ks][1] = live_g8 && in_k ? *reinterpret_cast<const uint32_t*>(q_g8 + 16 * ks + 2 * t) : 0u;
            q_a[ks][2] = live_g && in_k ? *reinterpret_cast<const uint32_t*>(q_g + 16 * ks + 8 + 2 * t) : 0u;
            q_a[ks][3] = live_g8 && in_k ? *reinterpret_cast<const uint32_t*>(q_g8 + 16 * ks + 8 + 2 * t) : 0u;
        }
    }
    const PooledWeight weight_of(scale, cap, head_bias != nullptr ? head_bias[head] : 0.0f);
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;

    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int stage = tile % kPooledMmaStages;
        load(tile + kPooledMmaStages - 1);   // into the stage that was used up in the turn before (the barrier at its end)
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kPooledMmaStages - 1) : "memory");
        __syncthreads();
        const bool pooled = tile < pooled_tiles;
        const int base = pooled ? tile * kPooledMmaKeys : (first_token_tile + tile - pooled_tiles) * kPooledMmaKeys;
        // a warp none of whose rows sees any of the tile's rows skips the arithmetic
        const int p_low = p_first + token_block * 16, p_high = min(p_last, p_low + 15);
        const bool any = !idle && (pooled ? base < (pool > 0 ? max(0, p_high - window + 1) / pool : 0) : (base <= p_high && base + kPooledMmaKeys - 1 + window > p_low));
        if (any) {
            const __nv_bfloat16* rows = pooled_rows + static_cast<size_t>(stage) * kPooledMmaKeys * pitch;
            float sc[kPooledMmaKeys / 8][4];
#pragma unroll
            for (int n = 0; n < kPooledMmaKeys / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
            // K as B operand, four 8 x 8 pieces at a time: rows 8 n (+8) x channels 16 ks (+8); lane l gives the address of row l % 8 of piece l / 8
            const __nv_bfloat16* k_rows = rows + static_cast<size_t>((lane & 7) + (lane >> 4) * 8) * pitch + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                if (16 * ks < L.dk) {
#pragma unroll
                    for (int n = 0; n < kPooledMmaKeys / 8; n += 2) {
                        uint32_t k_b[4];
                        pooled_ldmatrix_x4(k_b, k_rows + static_cast<size_t>(8 * n) * pitch + 16 * ks);
                        pooled_mma(sc[n], q_a[ks], k_b[0], k_b[1]);
                        pooled_mma(sc[n + 1], q_a[ks], k_b[2], k_b[3]);
                    }
                }
            }
            // a tile all of whose rows every one of the warp's 16 queries sees needs no mask (all its queries exist, then)
            const bool all_seen = token_block * 16 + 15 < count &&
                                  (pooled ? base + kPooledMmaKeys <= (pool > 0 ? max(0, p_low - window + 1) / pool : 0)
                                          : (base + kPooledMmaKeys - 1 <= p_low && base + window > p_low + 15));
            auto weigh = [&](auto capped_tag) {
                constexpr bool kCapped = decltype(capped_tag)::value;
                if (all_seen) {
#pragma unroll
                    for (int n = 0; n < kPooledMmaKeys / 8; ++n) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) sc[n][e] = weight_of.template value<kCapped>(sc[n][e]);
                    }
                } else {
#pragma unroll
                    for (int n = 0; n < kPooledMmaKeys / 8; ++n) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int where = base + 8 * n + 2 * t + (e & 1);
                            const bool upper = e < 2;   // row g; else row g + 8
                            const bool seen = pooled ? where < (upper ? seen_g : seen_g8)
                                                     : (upper ? (live_g && where <= p_g && where + window > p_g) : (live_g8 && where <= p_g8 && where + window > p_g8));
                            sc[n][e] = seen ? weight_of.template value<kCapped>(sc[n][e]) : 0.0f;
                        }
                    }
                }
            };
            if (weight_of.capped) weigh(std::true_type{}); else weigh(std::false_type{});
#pragma unroll
            for (int kk = 0; kk < kPooledMmaKeys / 16; ++kk) {
                uint32_t p_a[4];
                p_a[0] = pooled_pack(sc[2 * kk][0], sc[2 * kk][1]);
                p_a[1] = pooled_pack(sc[2 * kk][2], sc[2 * kk][3]);
                p_a[2] = pooled_pack(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                p_a[3] = pooled_pack(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
                // four 8 x 8 pieces of V at a time: keys 16 kk (+8) x channels 16 n (+8); lane l gives the address of row l % 8 of piece l / 8
                const __nv_bfloat16* v_rows = rows + static_cast<size_t>(16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + L.dk + (lane >> 4) * 8;
#pragma unroll
                for (int n = 0; n < DV / 16; ++n) {
                    if (16 * n < L.dv) {
                        uint32_t v_b[4];
                        pooled_ldmatrix_x4_trans(v_b, v_rows + 16 * n);
                        pooled_mma(o[2 * n], p_a, v_b[0], v_b[1]);
                        pooled_mma(o[2 * n + 1], p_a, v_b[2], v_b[3]);
                    }
                }
            }
        }
        __syncthreads();   // the stage is refilled in the next turn
    }
    if (idle) return;
    if (partial != nullptr) {
#pragma unroll
        for (int upper = 0; upper < 2; ++upper) {
            if (!(upper == 0 ? live_g : live_g8)) continue;
            float* destination = partial + ((static_cast<size_t>(blockIdx.z) * total_rows + first_row + (upper == 0 ? row_g : row_g8)) * heads + head) * L.dv;
#pragma unroll
            for (int n = 0; n < DV / 8; ++n)
                if (8 * n < L.dv) *reinterpret_cast<float2*>(destination + 8 * n + 2 * t) = make_float2(o[n][2 * upper], o[n][2 * upper + 1]);
        }
        return;
    }
    // turned back by the row's position, rounded once; o[n][0..1]: row g, channels 8 n + 2 t (+1); o[n][2..3]: row g + 8
    const int half_tiles = L.dv / 16;   // channel c and c + dv / 2 lie half_tiles tiles apart, in the same thread
#pragma unroll
    for (int upper = 0; upper < 2; ++upper) {
        if (!(upper == 0 ? live_g : live_g8)) continue;
        const float p = static_cast<float>(upper == 0 ? p_g : p_g8);
        __nv_bfloat16* destination = out + (static_cast<size_t>(first_row + (upper == 0 ? row_g : row_g8)) * heads + head) * L.dv;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            if (8 * n >= L.dv) continue;
            float low = o[n][2 * upper], high = o[n][2 * upper + 1];
            if (v_freq != nullptr) {
                float sine, cosine;
                if (v_interleaved) {
                    sincosf(p * v_freq[4 * n + t], &sine, &cosine);
                    const float a = low, b = high;
                    low = a * cosine + b * sine;
                    high = b * cosine - a * sine;
                } else {
                    const bool first_half = n < half_tiles;
                    const int partner = first_half ? n + half_tiles : n - half_tiles;
                    const int pair = 8 * (first_half ? n : partner) + 2 * t;
                    float other_low = 0.0f, other_high = 0.0f;
#pragma unroll
                    for (int m = 0; m < DV / 8; ++m)
                        if (m == partner) other_low = o[m][2 * upper], other_high = o[m][2 * upper + 1];
                    sincosf(p * v_freq[pair], &sine, &cosine);
                    const float turned_low = first_half ? low * cosine + other_low * sine : low * cosine - other_low * sine;
                    sincosf(p * v_freq[pair + 1], &sine, &cosine);
                    const float turned_high = first_half ? high * cosine + other_high * sine : high * cosine - other_high * sine;
                    low = turned_low, high = turned_high;
                }
            }
            *reinterpret_cast<uint32_t*>(destination + 8 * n + 2 * t) = pooled_pack(low, high);
        }
    }
}

// ---------------------------------------------------------------- single tokens (decoding) on the tensor cores
// A token that attends alone has one query a head, so the products are turned round: the rows of a product are 16 rows of the
// cache, its columns up to 16 query heads of one K/V head.  S^T = K Q^T (A: the rows' keys straight from shared memory, B: the
// queries from registers), the weights where the accumulators lie (four an element of a thread, not 32 as in a tile of tokens
// of which one row is real), P^T rounded and moved into the B operand's layout by `movmatrix`, O^T += V^T P^T with V^T through
// ldmatrix.trans.  Warps 0 to 3 take 16 of a block's 64 rows each (all eight warps copy); at the end their sums are added in warp
// order through shared memory, turned back and rounded (or left in 32-bit for `pooled_finish` where CTAs share a token's rows).
constexpr int kPooledSingleHeads = 16;   // query heads of one K/V head a CTA takes at most

__device__ __forceinline__ uint32_t pooled_movmatrix_trans(uint32_t value) {
    uint32_t result;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(result) : "r"(value));
    return result;
}

template <int DK, int DV>
__global__ void __launch_bounds__(32 * kPooledMmaWarps)
pooled_attention_single_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pages, const __nv_bfloat16* __restrict__ pooled_pages,
                               __nv_bfloat16* __restrict__ out, const int* __restrict__ singles, const int* __restrict__ positions,
                               const int* __restrict__ token_segment, const int* __restrict__ block_table, const int* __restrict__ pool_table,
                               PooledLayout L, int heads, float scale, float cap, const float* __restrict__ head_bias, int window, int pool,
                               const float* __restrict__ v_freq, int v_interleaved, int* status, float* __restrict__ partial, int total_rows) {
    extern __shared__ __align__(16) __nv_bfloat16 pooled_rows[];   // kPooledMmaStages stages of 64 rows of `pitch` elements; at the end the warps' sums
    const int row_width = L.dk + L.dv, pitch = row_width + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row = singles[blockIdx.x];
    const int per_group = heads / L.groups, head_parts = (per_group + kPooledSingleHeads - 1) / kPooledSingleHeads;
    const int group = blockIdx.y / head_parts, first_head = group * per_group + (blockIdx.y % head_parts) * kPooledSingleHeads;
    const int num_heads = min(kPooledSingleHeads, group * per_group + per_group - first_head);
    const int segment = token_segment[row];
    const int p_last = positions[row];
    const int blocks_seen = pool > 0 ? max(0, p_last - window + 1) / pool : 0;
    const int first_key = max(0, p_last - window + 1);
    const int pooled_tiles = (blocks_seen + kPooledMmaKeys - 1) / kPooledMmaKeys;
    const int first_token_tile = first_key / kPooledMmaKeys, token_tiles = p_last / kPooledMmaKeys - first_token_tile + 1;
    const int all_tiles = pooled_tiles + token_tiles;
    const int tile_begin = static_cast<int>(static_cast<long long>(all_tiles) * blockIdx.z / gridDim.z);
    const int tile_end = static_cast<int>(static_cast<long long>(all_tiles) * (blockIdx.z + 1) / gridDim.z);
    const int chunks = row_width / 8;
    const size_t group_offset = static_cast<size_t>(group) * row_width, row_stride = static_cast<size_t>(L.groups) * row_width;

    const int load_row = threadIdx.x >> 2, load_part = threadIdx.x & 3;
    auto lookup = [&](int tile) -> int {
        if (tile >= tile_end) return -1;
        const bool pooled = tile < pooled_tiles;
        const int where = (pooled ? tile * kPooledMmaKeys : (first_token_tile + tile - pooled_tiles) * kPooledMmaKeys) + load_row;
        if (!(pooled ? where < blocks_seen : (where >= first_key && where <= p_last))) return -1;
        const int page = pooled ? pooled_page(pool_table, L, segment, where) : token_page(block_table, L, segment, where);
        if (page < 0) report_error(status, kBadPage);
        return page;
    };
    int page_ahead = lookup(tile_begin);
    auto load = [&](int tile) {
        if (tile >= tile_end) {
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            return;
        }
        __nv_bfloat16* destination = pooled_rows + (static_cast<size_t>(tile % kPooledMmaStages) * kPooledMmaKeys + load_row) * pitch;
        const bool pooled = tile < pooled_tiles;
        const int where = (pooled ? tile * kPooledMmaKeys : (first_token_tile + tile - pooled_tiles) * kPooledMmaKeys) + load_row;
        const int page = page_ahead;
        const int per_page = pooled ? L.pool_rows : L.page_size;
        const __nv_bfloat16* source = (pooled ? pooled_pages : pages) + (page < 0 ? 0 : (static_cast<size_t>(page) * per_page + where % per_page) * row_stride + group_offset);
        for (int chunk = load_part; chunk < chunks; chunk += 4) pooled_copy_16(destination + 8 * chunk, source + 8 * chunk, page >= 0);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        page_ahead = lookup(tile + 1);
    };
#pragma unroll
    for (int ahead = 0; ahead < kPooledMmaStages - 1; ++ahead) load(tile_begin + ahead);

    // the queries as B operands: head tile n, column g is head first_head + 8 n + g
    constexpr int kHeadTiles = kPooledSingleHeads / 8;
    uint32_t q_b[DK / 16][kHeadTiles][2];
#pragma unroll
    for (int n = 0; n < kHeadTiles; ++n) {
        const bool real = 8 * n + g < num_heads;
        const __nv_bfloat16* q_head = q + (static_cast<size_t>(row) * heads + first_head + (real ? 8 * n + g : 0)) * L.dk;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            const bool in_k = real && 16 * ks < L.dk;
            q_b[ks][n][0] = in_k ? *reinterpret_cast<const uint32_t*>(q_head + 16 * ks + 2 * t) : 0u;
            q_b[ks][n][1] = in_k ? *reinterpret_cast<const uint32_t*>(q_head + 16 * ks + 8 + 2 * t) : 0u;
        }
    }
    // an accumulator's columns are heads 8 n + 2 t and 8 n + 2 t + 1: their biases
    float offsets[kHeadTiles][2];
    const PooledWeight weight_of(scale, cap, 0.0f);
#pragma unroll
    for (int n = 0; n < kHeadTiles; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int head = 8 * n + 2 * t + e;
            const float bias = head_bias != nullptr && head < num_heads ? head_bias[first_head + head] : 0.0f;
            offsets[n][e] = PooledWeight(scale, cap, bias).offset;
        }
    float o[DV / 16][kHeadTiles][4];   // rows: channels 16 m + g (+8); columns: heads 8 n + 2 t (+1)
#pragma unroll
    for (int m = 0; m < DV / 16; ++m)
#pragma unroll
        for (int n = 0; n < kHeadTiles; ++n) o[m][n][0] = o[m][n][1] = o[m][n][2] = o[m][n][3] = 0.0f;
    const bool second_tile = num_heads > 8;

    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int stage = tile % kPooledMmaStages;
        load(tile + kPooledMmaStages - 1);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kPooledMmaStages - 1) : "memory");
        __syncthreads();
        const bool pooled = tile < pooled_tiles;
        const int base = (pooled ? tile * kPooledMmaKeys : (first_token_tile + tile - pooled_tiles) * kPooledMmaKeys) + 16 * warp;   // the warp's 16 rows
        const bool any = warp < kPooledMmaKeys / 16 && (pooled ? base < blocks_seen : (base <= p_last && base + 15 >= first_key));
        if (any) {
            const __nv_bfloat16* rows = pooled_rows + (static_cast<size_t>(stage) * kPooledMmaKeys + 16 * warp) * pitch;
            float sc[kHeadTiles][4];
#pragma unroll
            for (int n = 0; n < kHeadTiles; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                if (16 * ks < L.dk) {
                    uint32_t k_a[4];
                    const __nv_bfloat16* k_row = rows + static_cast<size_t>(g) * pitch + 16 * ks + 2 * t;
                    k_a[0] = *reinterpret_cast<const uint32_t*>(k_row);
                    k_a[1] = *reinterpret_cast<const uint32_t*>(k_row + 8 * pitch);
                    k_a[2] = *reinterpret_cast<const uint32_t*>(k_row + 8);
                    k_a[3] = *reinterpret_cast<const uint32_t*>(k_row + 8 * pitch + 8);
                    pooled_mma(sc[0], k_a, q_b[ks][0][0], q_b[ks][0][1]);
                    if (second_tile) pooled_mma(sc[1], k_a, q_b[ks][1][0], q_b[ks][1][1]);
                }
            }
            // sc[n][0..1]: row g of the warp's 16; sc[n][2..3]: row g + 8
            const int where_low = base + g, where_high = base + g + 8;
            const bool seen_low = pooled ? where_low < blocks_seen : (where_low >= first_key && where_low <= p_last);
            const bool seen_high = pooled ? where_high < blocks_seen : (where_high >= first_key && where_high <= p_last);
            uint32_t p_b[kHeadTiles][2];
#pragma unroll
            for (int n = 0; n < kHeadTiles; ++n) {
                float w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x = weight_of.capped ? pooled_reciprocal(1.0f + pooled_exp2(sc[n][e] * weight_of.to_exponent)) : sc[n][e];
                    const float value = pooled_reciprocal(1.0f + pooled_exp2(fmaf(x, weight_of.slope, offsets[n][e & 1])));
                    w[e] = (e < 2 ? seen_low : seen_high) ? value : 0.0f;
                }
                // (row g, heads 2 t, 2 t + 1) -> (head g, rows 2 t, 2 t + 1): the B operand of the second product
                p_b[n][0] = pooled_movmatrix_trans(pooled_pack(w[0], w[1]));
                p_b[n][1] = pooled_movmatrix_trans(pooled_pack(w[2], w[3]));
            }
            // V^T as A operand: four 8 x 8 pieces, rows 0-7 / 8-15 of the warp's 16 x channels 16 m (+8); lane l gives row l % 8 of piece l / 8
            const __nv_bfloat16* v_rows = rows + static_cast<size_t>((lane & 7) + (lane >> 4) * 8) * pitch + L.dk + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int m = 0; m < DV / 16; ++m) {
                if (16 * m < L.dv) {
                    uint32_t v_a[4];
                    pooled_ldmatrix_x4_trans(v_a, v_rows + 16 * m);
                    pooled_mma(o[m][0], v_a, p_b[0][0], p_b[0][1]);
                    if (second_tile) pooled_mma(o[m][1], v_a, p_b[1][0], p_b[1][1]);
                }
            }
        }
        __syncthreads();
    }
    // the four warps' sums side by side in shared memory: [warp][channel][head]
    float* sums = reinterpret_cast<float*>(pooled_rows);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    if (warp < kPooledMmaKeys / 16) {
#pragma unroll
        for (int m = 0; m < DV / 16; ++m) {
            if (16 * m >= L.dv) continue;
#pragma unroll
            for (int n = 0; n < kHeadTiles; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int channel = 16 * m + g + (e >= 2 ? 8 : 0), head = 8 * n + 2 * t + (e & 1);
                    sums[(static_cast<size_t>(warp) * L.dv + channel) * kPooledSingleHeads + head] = o[m][n][e];
                }
            }
        }
    }
    __syncthreads();
    const int half = L.dv / 2;
    for (int index = threadIdx.x; index < num_heads * half; index += blockDim.x) {
        const int head = index / half, pair = index - head * half;
        const int first = v_interleaved ? 2 * pair : pair, second = v_interleaved ? 2 * pair + 1 : pair + half;
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int w = 0; w < kPooledMmaKeys / 16; ++w) {
            a += sums[(static_cast<size_t>(w) * L.dv + first) * kPooledSingleHeads + head];
            b += sums[(static_cast<size_t>(w) * L.dv + second) * kPooledSingleHeads + head];
        }
        const size_t offset = (static_cast<size_t>(row) * heads + first_head + head) * L.dv;
        if (partial != nullptr) {
            float* destination = partial + static_cast<size_t>(blockIdx.z) * total_rows * heads * L.dv + offset;
            destination[first] = a;
            destination[second] = b;
            continue;
        }
        if (v_freq != nullptr) {
            float sine, cosine;
            sincosf(static_cast<float>(p_last) * v_freq[pair], &sine, &cosine);
            const float turned = a * cosine + b * sine;
            b = b * cosine - a * sine;
            a = turned;
        }
        out[offset + first] = __float2bfloat16_rn(a);
        out[offset + second] = __float2bfloat16_rn(b);
    }
}

// grid (rows), a thread per head and pair of channels: out = the shares' sums added in order, turned back by the row's position.
// Only the rows the attention kernel before it wrote are finished: `rows` lists them, one a block (tokens that attend alone), or `tiles`
// does ((first row, count) a tile; grid (tiles, tokens a tile has at most)).
__global__ void pooled_finish_kernel(const float* __restrict__ partial, int shares, __nv_bfloat16* __restrict__ out, const int* __restrict__ positions,
                                     int total_rows, int heads, int dv, const float* __restrict__ v_freq, int v_interleaved, const int* __restrict__ rows,
                                     const int* __restrict__ tiles) {
    if (tiles != nullptr && static_cast<int>(blockIdx.y) >= tiles[2 * blockIdx.x + 1]) return;
    const int row = tiles != nullptr ? tiles[2 * blockIdx.x] + static_cast<int>(blockIdx.y) : rows[blockIdx.x];
    const float p = static_cast<float>(positions[row]);
    const size_t share_stride = static_cast<size_t>(total_rows) * heads * dv;
    for (int index = threadIdx.x; index < heads * (dv / 2); index += blockDim.x) {
        const int head = index / (dv / 2), pair = index - head * (dv / 2);
        const size_t offset = (static_cast<size_t>(row) * heads + head) * dv;
        const int first = v_interleaved ? 2 * pair : pair, second = v_interleaved ? 2 * pair + 1 : pair + dv / 2;
        float a = 0.0f, b = 0.0f;
        for (int share = 0; share < shares; ++share) {
            a += partial[share * share_stride + offset + first];
            b += partial[share * share_stride + offset + second];
        }
        if (v_freq != nullptr) {
            float sine, cosine;
            sincosf(p * v_freq[pair], &sine, &cosine);
            const float turned = a * cosine + b * sine;
            b = b * cosine - a * sine;
            a = turned;
        }
        out[offset + first] = __float2bfloat16_rn(a);
        out[offset + second] = __float2bfloat16_rn(b);
    }
}

}  // namespace lb

extern "C" {

int lb_pooled_rewrite(const void* qkv, int stride, void* q_out, void* pages, const float* qk_freq, int rot_dims, int qk_interleaved,
                      const float* v_freq, int v_interleaved, const int* positions, const int* token_segment, const int* block_table, int tokens,
                      int heads, int groups, int dk, int dv, int page_size, int num_pages, int max_blocks, int write_kv, int dtype, int* status,
                      cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (heads % groups != 0 || rot_dims < 0 || rot_dims > dk || rot_dims % 2 != 0 || (v_freq != nullptr && dv % 2 != 0)) return -2;
    lb::PooledLayout L{page_size, num_pages, max_blocks, 1, 0, 0, groups, dk, dv};
    LB_DISPATCH_DTYPE(dtype, {
        lb::pooled_rewrite_kernel<T><<<tokens, 256, 0, stream>>>(static_cast<const T*>(qkv), stride, static_cast<T*>(q_out), static_cast<T*>(pages), qk_freq, rot_dims, qk_interleaved, v_freq, v_interleaved, positions,
                                                                  token_segment, block_table, L, heads, write_kv, status);
    })
    return LB_LAUNCH_RESULT();
}

// max_length: the longest portion of the step (a portion of n tokens completes at most n / pool + 1 blocks).
int lb_pooled_means(const void* pages, void* pooled_pages, const int* segment_length, const int* segment_context,
                    const int* block_table, const int* pool_table, int segments, int max_length, int groups, int dk, int dv, int page_size, int num_pages,
                    int max_blocks, int pool_rows, int pool_pages, int pool_max_blocks, int pool, int dtype, int* status, cudaStream_t stream) {
    if (segments == 0 || max_length == 0) return 0;
    if (pool < 1 || pool_rows < 1) return -2;
    lb::PooledLayout L{page_size, num_pages, max_blocks, pool_rows, pool_pages, pool_max_blocks, groups, dk, dv};
    const dim3 grid(segments, max_length / pool + 1);
    LB_DISPATCH_DTYPE(dtype, {
        lb::pooled_means_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(pages), static_cast<T*>(pooled_pages), segment_length, segment_context, block_table, pool_table, L, pool, status);
    })
    return LB_LAUNCH_RESULT();
}

int lb_pooled_attention_plain(const void* q, const void* pages, const void* pooled_pages, void* out,
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
            static_cast<const T*>(q), static_cast<const T*>(pages), static_cast<const T*>(pooled_pages), static_cast<T*>(out), positions, token_segment, block_table, pool_table, L, heads, scale, cap, head_bias, window,
            pool, v_freq, v_interleaved, status);
    })
    return LB_LAUNCH_RESULT();
}

// head_block: the query heads of a K/V head that one CTA takes (1 to 4; its tiles have 16 * (8 / head_block) tokens at most).  shares > 1:
// that many CTAs share out a tile's rows; `partial` then holds shares x total_rows x heads x dv floats.
int lb_pooled_attention_mma(const void* q, const void* pages, const void* pooled_pages, void* out, const int* tiles, int num_tiles, const int* positions,
                            const int* token_segment, const int* block_table, const int* pool_table, int heads, int groups, int dk, int dv, int page_size,
                            int num_pages, int max_blocks, int pool_rows, int pool_pages, int pool_max_blocks, int head_block, float scale, float cap,
                            const float* head_bias, int window, int pool, const float* v_freq, int v_interleaved, int* status, cudaStream_t stream, int shares,
                            float* partial, int total_rows) {
    if (num_tiles == 0) return 0;
    if (shares < 1 || shares > 64 || (shares > 1 && partial == nullptr)) return -2;
    if (shares == 1) partial = nullptr;
    if (heads % groups != 0 || dk % 16 != 0 || dv % 16 != 0 || dk < 16 || dv < 16 || dk > 128 || dv > 128 || window < 1 || pool < 0 || head_block < 1 || head_block > 4) return -2;
    lb::PooledLayout L{page_size, num_pages, max_blocks, pool_rows > 0 ? pool_rows : 1, pool_pages, pool_max_blocks, groups, dk, dv};
    const int per_group = heads / groups;
    const dim3 grid(num_tiles, groups * ((per_group + head_block - 1) / head_block), shares);
    const size_t shared = static_cast<size_t>(lb::kPooledMmaStages) * lb::kPooledMmaKeys * (dk + dv + 8) * sizeof(__nv_bfloat16);
    const auto* q16 = static_cast<const __nv_bfloat16*>(q);
    const auto* pages16 = static_cast<const __nv_bfloat16*>(pages);
    const auto* pooled16 = static_cast<const __nv_bfloat16*>(pooled_pages);
    auto* out16 = static_cast<__nv_bfloat16*>(out);
    if (dk <= 64 && dv <= 64) {
        static lb::OncePerDevice once;
        lb::allow_shared_memory(once, lb::pooled_attention_mma_kernel<64, 64>, lb::kPooledMmaStages * lb::kPooledMmaKeys * (128 + 8) * 2);
        lb::pooled_attention_mma_kernel<64, 64><<<grid, 32 * lb::kPooledMmaWarps, shared, stream>>>(
            q16, pages16, pooled16, out16, tiles, positions, token_segment, block_table, pool_table, L, heads, head_block, scale, cap, head_bias, window, pool, v_freq,
            v_interleaved, status, partial, total_rows);
    } else {
        static lb::OncePerDevice once;
        lb::allow_shared_memory(once, lb::pooled_attention_mma_kernel<128, 128>, lb::kPooledMmaStages * lb::kPooledMmaKeys * (256 + 8) * 2);
        lb::pooled_attention_mma_kernel<128, 128><<<grid, 32 * lb::kPooledMmaWarps, shared, stream>>>(
            q16, pages16, pooled16, out16, tiles, positions, token_segment, block_table, pool_table, L, heads, head_block, scale, cap, head_bias, window, pool, v_freq,
            v_interleaved, status, partial, total_rows);
    }
    if (shares > 1)
        lb::pooled_finish_kernel<<<dim3(num_tiles, 16 * (lb::kPooledMmaWarps / head_block)), 256, 0, stream>>>(partial, shares, out16, positions, total_rows, heads, dv, v_freq,
                                                                                                            v_interleaved, nullptr, tiles);
    return LB_LAUNCH_RESULT();
}

// Tokens that attend alone: `singles` lists their rows.  shares > 1: that many CTAs share out a token's rows of the cache; `partial`
// then holds shares x total_rows x heads x dv floats (only the listed rows are written and read).
int lb_pooled_attention_single(const void* q, const void* pages, const void* pooled_pages, void* out, const int* singles, int num_singles, const int* positions,
                               const int* token_segment, const int* block_table, const int* pool_table, int heads, int groups, int dk, int dv, int page_size,
                               int num_pages, int max_blocks, int pool_rows, int pool_pages, int pool_max_blocks, float scale, float cap,
                               const float* head_bias, int window, int pool, const float* v_freq, int v_interleaved, int* status, cudaStream_t stream, int shares,
                               float* partial, int total_rows) {
    if (num_singles == 0) return 0;
    if (heads % groups != 0 || dk % 16 != 0 || dv % 16 != 0 || dk < 16 || dv < 16 || dk > 128 || dv > 128 || window < 1 || pool < 0) return -2;
    if (shares < 1 || shares > 64 || (shares > 1 && partial == nullptr)) return -2;
    if (shares == 1) partial = nullptr;
    lb::PooledLayout L{page_size, num_pages, max_blocks, pool_rows > 0 ? pool_rows : 1, pool_pages, pool_max_blocks, groups, dk, dv};
    const int per_group = heads / groups;
    const dim3 grid(num_singles, groups * ((per_group + lb::kPooledSingleHeads - 1) / lb::kPooledSingleHeads), shares);
    // the stages, and at the end four warps' sums of dv x 16 floats (no more than the stages)
    const size_t shared = static_cast<size_t>(lb::kPooledMmaStages) * lb::kPooledMmaKeys * (dk + dv + 8) * sizeof(__nv_bfloat16);
    const auto* q16 = static_cast<const __nv_bfloat16*>(q);
    const auto* pages16 = static_cast<const __nv_bfloat16*>(pages);
    const auto* pooled16 = static_cast<const __nv_bfloat16*>(pooled_pages);
    auto* out16 = static_cast<__nv_bfloat16*>(out);
    if (dk <= 64 && dv <= 64) {
        static lb::OncePerDevice once;
        lb::allow_shared_memory(once, lb::pooled_attention_single_kernel<64, 64>, lb::kPooledMmaStages * lb::kPooledMmaKeys * (128 + 8) * 2);
        lb::pooled_attention_single_kernel<64, 64><<<grid, 32 * lb::kPooledMmaWarps, shared, stream>>>(
            q16, pages16, pooled16, out16, singles, positions, token_segment, block_table, pool_table, L, heads, scale, cap, head_bias, window, pool, v_freq,
            v_interleaved, status, partial, total_rows);
    } else {
        static lb::OncePerDevice once;
        lb::allow_shared_memory(once, lb::pooled_attention_single_kernel<128, 128>, lb::kPooledMmaStages * lb::kPooledMmaKeys * (256 + 8) * 2);
        lb::pooled_attention_single_kernel<128, 128><<<grid, 32 * lb::kPooledMmaWarps, shared, stream>>>(
            q16, pages16, pooled16, out16, singles, positions, token_segment, block_table, pool_table, L, heads, scale, cap, head_bias, window, pool, v_freq,
            v_interleaved, status, partial, total_rows);
    }
    if (shares > 1)
        lb::pooled_finish_kernel<<<num_singles, 256, 0, stream>>>(partial, shares, out16, positions, total_rows, heads, dv, v_freq, v_interleaved, singles, nullptr);
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
