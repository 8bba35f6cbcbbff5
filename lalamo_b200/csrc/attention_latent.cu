// Latent attention: every token leaves one row [latent | rope] in its request's pages (the normed latent
// vector and one rotated key part shared by all heads).  A query head is given in the latent's space,
// [W_uk_h^T q_plain_h | rope(q_rot_h)], so that its score against a cached row is one dot product and the
// weighted sum of the rows' latent parts is what the head's value projection is applied to afterwards.
//
//   latent_prepare           norm of the latent, rotation of the shared key part and of the queries' rotated parts,
//                            the page write, and the queries laid out [token][head][latent | rope]
//   latent_attention_plain   one block per (token, head): 32-bit scores, softmax and sums; the 32-bit path's
//                            attention and the reference for the tensor-core kernel
//   gate_heads               heads' values [head][token][vdim] times sigmoid(gate), laid out [token][head * vdim]
//   heads_product            the two small products per head (queries into the latent's space, sums out of it, the latter with the gate)
#include "common.cuh"

namespace lb {

struct LatentLayout {
    int page_size;
    int num_pages;
    int max_blocks;   // columns of the block table
    int latent;       // channels of the normed latent vector (also the value a row stands for)
    int rope;         // channels of the rotated key part
};

template <typename T>
__device__ __forceinline__ T* latent_row(T* pages, const int* block_table, const LatentLayout& layout, int segment, int position) {
    const int block = position / layout.page_size;
    if (block >= layout.max_blocks) return nullptr;
    const int page = block_table[static_cast<size_t>(segment) * layout.max_blocks + block];
    if (page < 0 || page >= layout.num_pages) return nullptr;
    const size_t row = static_cast<size_t>(page) * layout.page_size + (position - block * layout.page_size);
    return pages + row * (layout.latent + layout.rope);
}

// grid (tokens, head blocks + 1): blocks (t, b) lay out token t's query heads, block (t, head blocks) writes the token's row.
//   q        [tokens][q_stride]: head h at h * (head_dim + rope), its last `rope` channels are rotated
//   q_latent [heads][tokens][latent]: the heads' unrotated parts taken into the latent's space
//   down     [tokens][down_stride]: [latent | rope]
//   q_out    [tokens][heads][latent + rope]
//   pages    [page][row][latent + rope]: row = [T(norm(down[:latent]) * (w + offset)) | rope(down[latent:])]
// The rotation pairs channel i with i + rope / 2: (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * inv_freq[i].
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ q_latent, const T* __restrict__ down, int down_stride,
                                      T* __restrict__ q_out, T* __restrict__ pages, const float* __restrict__ norm_weight, float eps, float scale_offset,
                                      const float* __restrict__ inv_freq, const int* __restrict__ positions, const int* __restrict__ token_segment,
                                      const int* __restrict__ block_table, LatentLayout layout, int tokens, int num_heads, int head_dim, int write_kv,
                                      int* status) {
    extern __shared__ float shared[];
    const int half = layout.rope / 2, latent = layout.latent, rope = layout.rope;
    float* cosines = shared;            // half
    float* sines = shared + half;       // half
    float* scratch = sines + half;      // 33
    // blocks (t, 0 .. head_blocks - 1) take heads_per_block heads each (one where the latent parts are copied, all where only
    // the rotated parts are written), block (t, head_blocks) the token's row
    const int token = blockIdx.x, unit = blockIdx.y, head_blocks = gridDim.y - 1, heads_per_block = (num_heads + head_blocks - 1) / head_blocks;
    if (unit == head_blocks && !write_kv) return;
    const int position = positions[token];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(static_cast<float>(position) * inv_freq[i], &sines[i], &cosines[i]);
    if (unit < head_blocks) {
        __syncthreads();
        const int head0 = unit * heads_per_block, heads_here = min(num_heads, head0 + heads_per_block) - head0;
        if (q_latent != nullptr) {   // null: whoever made them wrote them into q_out already
            for (int c = threadIdx.x; c < heads_here * latent; c += blockDim.x) {
                const int head = head0 + c / latent, d = c % latent;
                q_out[(static_cast<size_t>(token) * num_heads + head) * (latent + rope) + d] = q_latent[(static_cast<size_t>(head) * tokens + token) * latent + d];
            }
        }
        for (int c = threadIdx.x; c < heads_here * half; c += blockDim.x) {   // every pair of every head at once: one trip to memory
            const int head = head0 + c / half, i = c % half;
            const T* q_head = q + static_cast<size_t>(token) * q_stride + static_cast<size_t>(head) * (head_dim + rope) + head_dim;
            T* to = q_out + (static_cast<size_t>(token) * num_heads + head) * (latent + rope) + latent;
            const float u = to_float(q_head[i]), v = to_float(q_head[half + i]);
            to[i] = from_float<T>(u * cosines[i] - v * sines[i]);
            to[half + i] = from_float<T>(v * cosines[i] + u * sines[i]);
        }
        return;
    }
    const T* row = down + static_cast<size_t>(token) * down_stride;
    float squares = 0.0f;
    for (int d = threadIdx.x; d < latent; d += blockDim.x) {
        const float v = to_float(row[d]);
        squares += v * v;
    }
    const float total = block_sum(squares, scratch);   // also orders the writes to cosines[] and sines[]
    T* dst = latent_row(pages, block_table, layout, token_segment[token], position);
    if (dst == nullptr) {
        if (threadIdx.x == 0) report_error(status, kBadPage);
        return;
    }
    const float inv = rsqrtf(total / static_cast<float>(latent) + eps);
    for (int d = threadIdx.x; d < latent; d += blockDim.x) dst[d] = from_float<T>(to_float(row[d]) * inv * (norm_weight[d] + scale_offset));
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float u = to_float(row[latent + i]), v = to_float(row[latent + half + i]);
        dst[latent + i] = from_float<T>(u * cosines[i] - v * sines[i]);
        dst[latent + half + i] = from_float<T>(v * cosines[i] + u * sines[i]);
    }
}

constexpr int kLatentThreads = 128, kLatentChunk = 128, kLatentMaxDimsPerThread = 8;   // latent <= 1024

// grid (tokens, heads).  The query at position p sees the rows j with max(0, p - window + 1) <= j <= p (window <= 0:
// all j <= p).  Rows are visited in chunks that start at the first visible row, so the result does not depend on how a
// prompt was cut into steps or on what else is in the batch.  out [tokens][heads][latent].
template <typename T>
__global__ void latent_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pages, T* __restrict__ out, const int* __restrict__ positions,
                                              const int* __restrict__ token_segment, const int* __restrict__ block_table, LatentLayout layout, int num_heads,
                                              float scale, int window, int* status, const float* __restrict__ sink) {
    // sink (may be null): one number per head whose exponential joins the denominator; it has no row and is not scaled.
    extern __shared__ __align__(16) float shared[];
    const int latent = layout.latent, full = layout.latent + layout.rope;
    const T** rows = reinterpret_cast<const T**>(shared);                       // kLatentChunk pointers
    float* scores = shared + 2 * kLatentChunk;                                   // kLatentChunk
    float* scratch = scores + kLatentChunk;                                      // 33 (+ 3 to keep q_shared apart)
    float* q_shared = scratch + 36;                                              // full
    const int token = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int segment = token_segment[token];
    const int position = positions[token];
    const int first = window > 0 ? max(0, position - window + 1) : 0;
    const T* q_row = q + (static_cast<size_t>(token) * num_heads + head) * full;
    for (int d = tid; d < full; d += blockDim.x) q_shared[d] = to_float(q_row[d]);
    __syncthreads();

    float acc[kLatentMaxDimsPerThread];
#pragma unroll
    for (int i = 0; i < kLatentMaxDimsPerThread; ++i) acc[i] = 0.0f;
    float running_max = -INFINITY, running_sum = 0.0f;
    for (int chunk = first; chunk <= position; chunk += kLatentChunk) {
        const int count = min(kLatentChunk, position + 1 - chunk);
        float local_max = -INFINITY;
        for (int i = warp; i < count; i += kLatentThreads / 32) {   // a warp per row, lanes along its channels
            const T* row = latent_row(const_cast<T*>(pages), block_table, layout, segment, chunk + i);
            float s = -INFINITY;
            if (row == nullptr) {
                if (lane == 0) report_error(status, kBadPage);
            } else {
                float dot = 0.0f;
                for (int d = lane; d < full; d += 32) dot += q_shared[d] * to_float(row[d]);
                s = warp_sum(dot) * scale;
            }
            if (lane == 0) {
                rows[i] = row;
                scores[i] = s;
            }
            local_max = fmaxf(local_max, s);
        }
        const float chunk_max = block_max(local_max, scratch);
        const float new_max = fmaxf(running_max, chunk_max);
        const float rescale = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
        float local_sum = 0.0f;
        for (int i = tid; i < count; i += blockDim.x) {
            const float p = new_max == -INFINITY || rows[i] == nullptr ? 0.0f : expf(scores[i] - new_max);
            scores[i] = p;
            local_sum += p;
        }
        const float chunk_sum = block_sum(local_sum, scratch);   // also orders the writes to scores[]
        running_sum = running_sum * rescale + chunk_sum;
        running_max = new_max;
#pragma unroll
        for (int slot = 0; slot < kLatentMaxDimsPerThread; ++slot) {
            const int d = tid + slot * kLatentThreads;
            if (d < latent) {
                float sum = acc[slot] * rescale;
                for (int i = 0; i < count; ++i) {
                    const float p = scores[i];
                    if (p != 0.0f) sum += p * to_float(rows[i][d]);
                }
                acc[slot] = sum;
            }
        }
        __syncthreads();   // scores[] and rows[] are rewritten by the next chunk
    }
    T* dst = out + (static_cast<size_t>(token) * num_heads + head) * latent;
    if (sink != nullptr) {
        // sum_j e^(s_j - m) + e^(sink - m), with both scaled by e^(m - sink) where the sink is the larger
        const float gap = sink[head] - running_max;
        if (gap > 0.0f) {
            const float shrink = expf(-gap);
#pragma unroll
            for (int slot = 0; slot < kLatentMaxDimsPerThread; ++slot) acc[slot] *= shrink;
            running_sum = running_sum * shrink + 1.0f;
        } else {
            running_sum += expf(gap);
        }
    }
    const float norm = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
#pragma unroll
    for (int slot = 0; slot < kLatentMaxDimsPerThread; ++slot) {
        const int d = tid + slot * kLatentThreads;
        if (d < latent) dst[d] = from_float<T>(acc[slot] * norm);
    }
}

// out[t][h * vdim + j] = T(values[h][t][j] * sigmoid(gate[t * gate_stride + h * vdim + j]))   (gate null: no gate)
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ values, const T* __restrict__ gate, int gate_stride, T* __restrict__ out, int tokens, int num_heads,
                                  int value_dim) {
    const int token = blockIdx.x, width = num_heads * value_dim;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const int head = c / value_dim, j = c - head * value_dim;
        float v = to_float(values[(static_cast<size_t>(head) * tokens + token) * value_dim + j]);
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-to_float(gate[static_cast<size_t>(token) * gate_stride + c])));
        out[static_cast<size_t>(token) * width + c] = from_float<T>(v);
    }
}


// ------------------------------------------------------------------------------- tensor cores
// The same attention on mma.sync (bfloat16, 32-bit accumulation) for latent + rope and latent multiples of 16.
//
// A CTA of four warps takes one item: up to 64 query rows = consecutive tokens of one request x a block of heads,
// 16 rows a warp.  All rows share the cached rows (there is one "key head"), which come through shared memory in blocks
// of 64 rows (cp.async, two buffers) that start at multiples of 64 from the request's first token, so the order of a
// query's sums does not depend on how the prompt was cut or on what shares its CTA.  A block serves both products: as
// K for S = Q K^T over latent + rope channels (ldmatrix), and, its first `latent` channels, as V for O += P V
// (ldmatrix.trans).  Rows that no query of the item sees are zero-filled, never read.  grid.z shares out the latent's
// channels in chunks of CHUNK (128, or 256 for latents wider than 128; every chunk computes the scores again); grid.y = head blocks x key splits: with splits > 1
// every CTA takes a share of the item's blocks and leaves (maximum, sum, unnormalised O) for latent_merge_kernel.
constexpr int kLatentMmaRows = 64, kLatentMmaKeys = 64, kLatentMmaThreads = 128;

struct LatentMmaParams {
    const __nv_bfloat16* q;       // [tokens][heads][latent + rope]
    const __nv_bfloat16* pages;   // [page][row][latent + rope]
    __nv_bfloat16* out;           // [tokens][heads][latent]
    float* partial;               // splits > 1: [tokens][heads][split][latent + 2] (O unnormalised, maximum in base-2 units, sum)
    const int* items;             // [num_items][2]: first token row, count
    const int* positions;
    const int* token_segment;
    const int* block_table;
    LatentLayout layout;
    int num_heads, heads_per_cta, tokens_per_cta, head_blocks, splits, window;
    float scale_log2;
    int* status;
    const float* sink;            // [heads] or null: a number per head whose exponential joins the denominator (not scaled)
};

__device__ __forceinline__ void latent_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* shared_address) {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(shared_address));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* shared_address) {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(shared_address));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

// 16 bytes from global to shared memory, or 16 zero bytes (nothing is read) if `valid` is false.
__device__ __forceinline__ void latent_copy_16(void* shared_destination, const void* global_source, bool valid) {
    const uint32_t destination = static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(destination), "l"(global_source), "r"(bytes) : "memory");
}

__device__ __forceinline__ float latent_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t latent_pack(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

template <int CHUNK>
__global__ void __launch_bounds__(kLatentMmaThreads)
latent_attention_mma_kernel(LatentMmaParams p) {
    constexpr int kLatentMmaChunk = CHUNK;
    extern __shared__ __align__(16) unsigned char latent_shared[];
    const int latent = p.layout.latent, full = p.layout.latent + p.layout.rope;
    const int pitch = full + 8;   // elements: rows 16 bytes apart modulo 128, so that ldmatrix meets no bank twice
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(latent_shared);          // [64][pitch]
    __nv_bfloat16* k_s = q_s + kLatentMmaRows * pitch;                             // [2][64][pitch]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int item = gridDim.x - 1 - blockIdx.x;   // a prompt's last items see the most rows: they start first
    const int head_block = blockIdx.y / p.splits, split = blockIdx.y - head_block * p.splits;
    const int chunk0 = blockIdx.z * kLatentMmaChunk;
    const int chunk = min(kLatentMmaChunk, latent - chunk0);   // a multiple of 16
    const int first_token = p.items[2 * item], count = p.items[2 * item + 1];
    const int head0 = head_block * p.heads_per_cta;
    const int heads_here = min(p.heads_per_cta, p.num_heads - head0);
    const int rows_used = count * heads_here;
    const int segment = p.token_segment[first_token];
    const int position0 = p.positions[first_token];
    const int last_position = position0 + count - 1;
    const int lowest = p.window > 0 ? max(0, position0 - p.window + 1) : 0;   // the lowest row any query of the item sees
    // this CTA's share of the item's blocks of 64 rows
    const int block_lo = lowest / kLatentMmaKeys, block_hi = last_position / kLatentMmaKeys + 1;
    const int per_split = (block_hi - block_lo + p.splits - 1) / p.splits;
    const int block_begin = block_lo + split * per_split, block_end = min(block_hi, block_begin + per_split);

    // queries: row r = (token r / heads_here, head head0 + r % heads_here); rows past rows_used are zero
    const int chunks_per_row = full / 8;
    // a thread's pieces are 128 apart: (row, piece within the row) advance by these steps
    const int row_step = kLatentMmaThreads / chunks_per_row, piece_step = kLatentMmaThreads - row_step * chunks_per_row;
    const int first_r = tid / chunks_per_row, first_piece = tid - first_r * chunks_per_row;
    for (int r = first_r, piece = first_piece; r < kLatentMmaRows;) {
        const bool valid = r < rows_used;
        const int token = first_token + (valid ? r / heads_here : 0), head = head0 + (valid ? r % heads_here : 0);
        latent_copy_16(q_s + r * pitch + piece * 8, p.q + (static_cast<size_t>(token) * p.num_heads + head) * full + piece * 8, valid);
        r += row_step;
        piece += piece_step;
        if (piece >= chunks_per_row) {
            piece -= chunks_per_row;
            ++r;
        }
    }
    auto load_block = [&](int block, int stage) {
        __nv_bfloat16* dst = k_s + stage * kLatentMmaKeys * pitch;
        const int key0 = block * kLatentMmaKeys;
        for (int r = first_r, piece = first_piece; r < kLatentMmaKeys;) {
            const int key = key0 + r;
            bool valid = key >= lowest && key <= last_position;
            const __nv_bfloat16* src = p.pages;
            if (valid) {
                const int table_column = key / p.layout.page_size;
                const int page = table_column < p.layout.max_blocks ? p.block_table[static_cast<size_t>(segment) * p.layout.max_blocks + table_column] : -1;
                if (page < 0 || page >= p.layout.num_pages) {
                    if (piece == 0) report_error(p.status, kBadPage);
                    valid = false;
                } else {
                    src = p.pages + (static_cast<size_t>(page) * p.layout.page_size + (key - table_column * p.layout.page_size)) * full + piece * 8;
                }
            }
            latent_copy_16(dst + r * pitch + piece * 8, src, valid);
            r += row_step;
            piece += piece_step;
            if (piece >= chunks_per_row) {
                piece -= chunks_per_row;
                ++r;
            }
        }
    };
    if (block_begin < block_end) load_block(block_begin, 0);
    asm volatile("cp.async.commit_group;\n" ::: "memory");

    const int g = lane >> 2, t = lane & 3;
    const int row_a = warp * 16 + g, row_b = row_a + 8;   // this thread's two rows of the CTA's 64
    const bool warp_active = warp * 16 < rows_used;
    const int position_a = position0 + (row_a < rows_used ? row_a / heads_here : 0);
    const int position_b = position0 + (row_b < rows_used ? row_b / heads_here : 0);
    const int first_a = p.window > 0 ? max(0, position_a - p.window + 1) : 0;
    const int first_b = p.window > 0 ? max(0, position_b - p.window + 1) : 0;
    const int last_first = p.window > 0 ? max(0, last_position - p.window + 1) : 0;   // the first row the item's last query sees
    float o[kLatentMmaChunk / 8][4];
#pragma unroll
    for (int j = 0; j < kLatentMmaChunk / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float max_a = -INFINITY, max_b = -INFINITY, sum_a = 0.0f, sum_b = 0.0f;   // maxima of the raw scores

    for (int block = block_begin; block < block_end; ++block) {
        const int stage = (block - block_begin) & 1;
        if (block + 1 < block_end) load_block(block + 1, stage ^ 1);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        __syncthreads();
        if (warp_active) {
            const __nv_bfloat16* k_block = k_s + stage * kLatentMmaKeys * pitch;
            float s[kLatentMmaKeys / 8][4];
#pragma unroll
            for (int j = 0; j < kLatentMmaKeys / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
            // a step's fragments are asked for before the step before's products are issued
            const __nv_bfloat16* a_address = q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (lane >> 4) * 8;
            const __nv_bfloat16* b_address = k_block + ((lane & 7) + (lane >> 4) * 8) * pitch + ((lane >> 3) & 1) * 8;
            uint32_t a[2][4], b[2][kLatentMmaKeys / 16][4];
            ldmatrix_x4(a[0], a_address);
#pragma unroll
            for (int j = 0; j < kLatentMmaKeys / 16; ++j) ldmatrix_x4(b[0][j], b_address + j * 16 * pitch);
            for (int k0 = 0; k0 < full; k0 += 32) {
                if (k0 + 16 < full) {
                    ldmatrix_x4(a[1], a_address + k0 + 16);
#pragma unroll
                    for (int j = 0; j < kLatentMmaKeys / 16; ++j) ldmatrix_x4(b[1][j], b_address + j * 16 * pitch + k0 + 16);
                }
#pragma unroll
                for (int j = 0; j < kLatentMmaKeys / 16; ++j) {
                    latent_mma(s[2 * j], a[0], b[0][j][0], b[0][j][1]);
                    latent_mma(s[2 * j + 1], a[0], b[0][j][2], b[0][j][3]);
                }
                if (k0 + 16 < full) {
                    if (k0 + 32 < full) {
                        ldmatrix_x4(a[0], a_address + k0 + 32);
#pragma unroll
                        for (int j = 0; j < kLatentMmaKeys / 16; ++j) ldmatrix_x4(b[0][j], b_address + j * 16 * pitch + k0 + 32);
                    }
#pragma unroll
                    for (int j = 0; j < kLatentMmaKeys / 16; ++j) {
                        latent_mma(s[2 * j], a[1], b[1][j][0], b[1][j][1]);
                        latent_mma(s[2 * j + 1], a[1], b[1][j][2], b[1][j][3]);
                    }
                }
            }
            // masks (only in blocks that reach past the item's first query or before its last query's window), and the
            // block's maxima per row
            const int key0 = block * kLatentMmaKeys;
            float block_max_a = -INFINITY, block_max_b = -INFINITY;
            if (key0 + kLatentMmaKeys - 1 > position0 || key0 < last_first) {
#pragma unroll
                for (int j = 0; j < kLatentMmaKeys / 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + 8 * j + 2 * t + e;
                        if (key < first_a || key > position_a) s[j][e] = -INFINITY;
                        if (key < first_b || key > position_b) s[j][2 + e] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < kLatentMmaKeys / 8; ++j) {
                block_max_a = fmaxf(block_max_a, fmaxf(s[j][0], s[j][1]));
                block_max_b = fmaxf(block_max_b, fmaxf(s[j][2], s[j][3]));
            }
            block_max_a = fmaxf(block_max_a, __shfl_xor_sync(0xffffffffu, block_max_a, 1));
            block_max_a = fmaxf(block_max_a, __shfl_xor_sync(0xffffffffu, block_max_a, 2));
            block_max_b = fmaxf(block_max_b, __shfl_xor_sync(0xffffffffu, block_max_b, 1));
            block_max_b = fmaxf(block_max_b, __shfl_xor_sync(0xffffffffu, block_max_b, 2));
            const float new_a = fmaxf(max_a, block_max_a), new_b = fmaxf(max_b, block_max_b);
            const float shift_a = new_a == -INFINITY ? 0.0f : new_a * p.scale_log2, shift_b = new_b == -INFINITY ? 0.0f : new_b * p.scale_log2;
            const float keep_a = max_a == -INFINITY ? 0.0f : latent_exp2(max_a * p.scale_log2 - shift_a);
            const float keep_b = max_b == -INFINITY ? 0.0f : latent_exp2(max_b * p.scale_log2 - shift_b);
            max_a = new_a;
            max_b = new_b;
            float add_a = 0.0f, add_b = 0.0f;
            uint32_t prob[kLatentMmaKeys / 16][4];   // P as the second product's first operand
#pragma unroll
            for (int j = 0; j < kLatentMmaKeys / 8; ++j) {
                const float p0 = latent_exp2(s[j][0] * p.scale_log2 - shift_a), p1 = latent_exp2(s[j][1] * p.scale_log2 - shift_a);
                const float p2 = latent_exp2(s[j][2] * p.scale_log2 - shift_b), p3 = latent_exp2(s[j][3] * p.scale_log2 - shift_b);
                // the sums add what the product uses: the rounded probabilities
                const __nv_bfloat162 low = __floats2bfloat162_rn(p0, p1), high = __floats2bfloat162_rn(p2, p3);
                add_a += __low2float(low) + __high2float(low);
                add_b += __low2float(high) + __high2float(high);
                prob[j >> 1][(j & 1) * 2] = *reinterpret_cast<const uint32_t*>(&low);
                prob[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&high);
            }
            sum_a = sum_a * keep_a + add_a;
            sum_b = sum_b * keep_b + add_b;
            if (__any_sync(0xffffffffu, keep_a != 1.0f || keep_b != 1.0f)) {   // no row's maximum moved: nothing to rescale
#pragma unroll
                for (int j = 0; j < kLatentMmaChunk / 8; ++j) {
                    o[j][0] *= keep_a;
                    o[j][1] *= keep_a;
                    o[j][2] *= keep_b;
                    o[j][3] *= keep_b;
                }
            }
            const __nv_bfloat16* v_address = k_block + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + chunk0 + (lane >> 4) * 8;
#pragma unroll
            for (int kk = 0; kk < kLatentMmaKeys / 16; ++kk) {
#pragma unroll
                for (int j = 0; j < kLatentMmaChunk / 16; j += 4) {   // four loads on their way before their products
                    uint32_t v[4][4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (16 * (j + u) < chunk) ldmatrix_x4_trans(v[u], v_address + kk * 16 * pitch + (j + u) * 16);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (16 * (j + u) < chunk) {
                            latent_mma(o[2 * (j + u)], prob[kk], v[u][0], v[u][1]);
                            latent_mma(o[2 * (j + u) + 1], prob[kk], v[u][2], v[u][3]);
                        }
                    }
                }
            }
        }
        __syncthreads();   // the buffer is reloaded by the next round's copies
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (!warp_active) return;
    // a row's sum lies in the four lanes of its quad
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half == 0 ? row_a : row_b;
        if (row >= rows_used) continue;
        const int token = first_token + row / heads_here, head = head0 + row % heads_here;
        const float sum = half == 0 ? sum_a : sum_b, top = half == 0 ? max_a : max_b;
        if (p.splits == 1) {
            float norm = sum > 0.0f ? 1.0f / sum : 0.0f;
            if (p.sink != nullptr) {
                // sum is relative to the largest score: sum_j 2^((s_j - top) scale_log2); the sink joins it as 2^(sink log2 e - top scale_log2),
                // computed on the side that cannot overflow
                const float gap = p.sink[head] * 1.4426950408889634f - (top == -INFINITY ? 0.0f : top * p.scale_log2);
                norm = top == -INFINITY ? 0.0f : (gap > 0.0f ? exp2f(-gap) / (sum * exp2f(-gap) + 1.0f) : 1.0f / (sum + exp2f(gap)));
            }
            __nv_bfloat16* dst = p.out + (static_cast<size_t>(token) * p.num_heads + head) * latent + chunk0;
#pragma unroll
            for (int j = 0; j < kLatentMmaChunk / 8; ++j)
                if (8 * j < chunk) *reinterpret_cast<uint32_t*>(dst + 8 * j + 2 * t) = latent_pack(o[j][2 * half] * norm, o[j][2 * half + 1] * norm);
        } else {
            float* dst = p.partial + ((static_cast<size_t>(token) * p.num_heads + head) * p.splits + split) * (latent + 2);
#pragma unroll
            for (int j = 0; j < kLatentMmaChunk / 8; ++j)
                if (8 * j < chunk) *reinterpret_cast<float2*>(dst + chunk0 + 8 * j + 2 * t) = make_float2(o[j][2 * half], o[j][2 * half + 1]);
            if (t == 0 && blockIdx.z == 0) {
                dst[latent] = top == -INFINITY ? -INFINITY : top * p.scale_log2;
                dst[latent + 1] = sum;
            }
        }
    }
}

// out[token][head] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s over the splits, in split order.  One block per (token, head);
// shared memory: a float per split.
__global__ void latent_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int splits, int latent,
                                    const float* __restrict__ sink, int num_heads) {
    extern __shared__ float split_weight[];
    const size_t row = blockIdx.x;
    const float* mine = partial + row * splits * (latent + 2);
    if (threadIdx.x < 32) {
        float top = -INFINITY;
        for (int s = threadIdx.x; s < splits; s += 32) top = fmaxf(top, mine[s * (latent + 2) + latent]);
        top = warp_max(top);
        // the sink (a number per head, base e, joined to the denominator once) counts as one more split with sum 1 and no rows
        const float sink_top = sink != nullptr ? sink[row % num_heads] * 1.4426950408889634f : -INFINITY;
        top = fmaxf(top, sink_top);
        for (int s = threadIdx.x; s < splits; s += 32) {
            const float m = mine[s * (latent + 2) + latent];
            split_weight[s] = m == -INFINITY ? 0.0f : exp2f(m - top);
        }
        __syncwarp();
        if (threadIdx.x == 0) {
            float total = sink != nullptr ? exp2f(sink_top - top) : 0.0f;
            for (int s = 0; s < splits; ++s) total += split_weight[s] * mine[s * (latent + 2) + latent + 1];   // in split order
            const float norm = total > 0.0f ? 1.0f / total : 0.0f;
            for (int s = 0; s < splits; ++s) split_weight[s] *= norm;
        }
    }
    __syncthreads();
    for (int d = threadIdx.x; d < latent; d += blockDim.x) {
        float sum = 0.0f;
#pragma unroll 4
        for (int s = 0; s < splits; ++s) sum += split_weight[s] * mine[s * (latent + 2) + d];   // a split that saw nothing left zeros
        out[row * latent + d] = __float2bfloat16_rn(sum);
    }
}


// ------------------------------------------------------------------ one small product per head
// out[t][h][n] = sum_k a[t][h][k] * B_h[k][n] for every head h, with B_h stored [K][N] (B_KN: a head's key projection, which takes
// the unrotated query channels into the latent's space) or [N][K] (a head's value projection applied to the summed rows), optionally
// times sigmoid(gate[t][h][n]).  Rows of a, out and gate are addressed by a token stride and a head stride, so inputs may be column
// slices of a wider product and the output a part of wider rows.  grid (blocks of 64 tokens, heads, blocks of 64 columns), four warps
// of 16 tokens; the tokens' rows and the columns' part of the head's matrix lie in shared memory; bfloat16, mma.sync with 32-bit sums;
// K and N multiples of 16.
struct HeadsProductParams {
    const __nv_bfloat16* a;
    long long a_token_stride;
    int a_head_stride;
    const __nv_bfloat16* b;
    __nv_bfloat16* out;
    long long out_token_stride;
    int out_head_stride;
    const __nv_bfloat16* gate;   // or null
    long long gate_token_stride;
    int gate_head_stride;
    int tokens, k, n;
    int blocks_per_cta;   // blocks of 64 columns a CTA takes
};

template <bool B_KN>
__global__ void __launch_bounds__(128)
heads_product_kernel(HeadsProductParams p) {
    extern __shared__ __align__(16) unsigned char product_shared[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, head = blockIdx.y, token0 = blockIdx.x * 64;
    // grid.z shares out the blocks of 64 columns; a CTA takes blocks_per_cta neighbouring blocks, whose part of the head's matrix it loads at once
    const int first_column = blockIdx.z * p.blocks_per_cta * 64, share = min(p.blocks_per_cta * 64, p.n - first_column);
    const int a_pitch = p.k + 8, b_pitch = (B_KN ? p.blocks_per_cta * 64 : p.k) + 8;
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(product_shared);   // [64][k + 8]
    __nv_bfloat16* b_s = a_s + 64 * a_pitch;                                   // [k][share + 8] or [share][k + 8]
    const int a_pieces = p.k / 8;
    const int rows_here = min(64, p.tokens - token0);
    for (int c = tid; c < rows_here * a_pieces; c += 128) {
        const int r = c / a_pieces, piece = c - r * a_pieces;
        latent_copy_16(a_s + r * a_pitch + piece * 8, p.a + static_cast<size_t>(token0 + r) * p.a_token_stride + static_cast<size_t>(head) * p.a_head_stride + piece * 8, true);
    }
    {
        const int b_rows = B_KN ? p.k : share, b_pieces = (B_KN ? share : p.k) / 8, b_global_pitch = B_KN ? p.n : p.k;
        const __nv_bfloat16* b_head = p.b + static_cast<size_t>(head) * p.k * p.n + (B_KN ? first_column : static_cast<size_t>(first_column) * p.k);
        for (int c = tid; c < b_rows * b_pieces; c += 128) {
            const int r = c / b_pieces, piece = c - r * b_pieces;
            latent_copy_16(b_s + r * b_pitch + piece * 8, b_head + static_cast<size_t>(r) * b_global_pitch + piece * 8, true);
        }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    if (warp * 16 >= rows_here) return;   // (rows past the tokens hold whatever shared memory held: their results are not stored)
    const int g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* a_address = a_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * a_pitch + (lane >> 4) * 8;
    for (int local = 0; local < share; local += 64) {
        const int n0 = first_column + local, columns = min(64, share - local);   // a multiple of 16
        float acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        for (int k0 = 0; k0 < p.k; k0 += 16) {
            uint32_t a[4], b[4][4];
            ldmatrix_x4(a, a_address + k0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (16 * j < columns) {
                    if constexpr (B_KN) ldmatrix_x4_trans(b[j], b_s + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * b_pitch + local + j * 16 + (lane >> 4) * 8);
                    else ldmatrix_x4(b[j], b_s + (local + j * 16 + (lane & 7) + (lane >> 4) * 8) * b_pitch + k0 + ((lane >> 3) & 1) * 8);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (16 * j < columns) {
                    latent_mma(acc[2 * j], a, b[j][0], b[j][1]);
                    latent_mma(acc[2 * j + 1], a, b[j][2], b[j][3]);
                }
            }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int token = token0 + warp * 16 + g + 8 * half;
            if (token >= p.tokens) continue;
            __nv_bfloat16* dst = p.out + static_cast<size_t>(token) * p.out_token_stride + static_cast<size_t>(head) * p.out_head_stride + n0;
            const __nv_bfloat16* gate = p.gate ? p.gate + static_cast<size_t>(token) * p.gate_token_stride + static_cast<size_t>(head) * p.gate_head_stride + n0 : nullptr;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (8 * j >= columns) continue;
                float low = acc[j][2 * half], high = acc[j][2 * half + 1];
                if (gate != nullptr) {
                    const float2 z = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + 8 * j + 2 * t));
                    // the product is rounded as it would be stored, then gated
                    low = __bfloat162float(__float2bfloat16_rn(low)) / (1.0f + expf(-z.x));
                    high = __bfloat162float(__float2bfloat16_rn(high)) / (1.0f + expf(-z.y));
                }
                *reinterpret_cast<uint32_t*>(dst + 8 * j + 2 * t) = latent_pack(low, high);
            }
        }
    }
}

}  // namespace lb

extern "C" {

int lb_latent_prepare(const void* q, int q_stride, const void* q_latent, const void* down, int down_stride, void* q_out, void* pages,
                      const float* norm_weight, float eps, float scale_offset, const float* inv_freq, const int* positions, const int* token_segment,
                      const int* block_table, int tokens, int num_heads, int head_dim, int latent, int rope, int page_size, int num_pages, int max_blocks,
                      int write_kv, int dtype, int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (rope < 0 || rope % 2 != 0 || latent < 1 || num_heads < 1) return -2;
    lb::LatentLayout layout{page_size, num_pages, max_blocks, latent, rope};
    const size_t shared = (static_cast<size_t>(rope) + 33) * sizeof(float);
    if (shared > 48 * 1024) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        lb::latent_prepare_kernel<T><<<dim3(tokens, (q_latent != nullptr ? num_heads : 1) + 1), q_latent != nullptr ? 64 : 128, shared, stream>>>(
            static_cast<const T*>(q), q_stride, static_cast<const T*>(q_latent), static_cast<const T*>(down), down_stride, static_cast<T*>(q_out),
            static_cast<T*>(pages), norm_weight, eps, scale_offset, inv_freq, positions, token_segment, block_table, layout, tokens, num_heads, head_dim,
            write_kv, status);
    })
    return LB_LAUNCH_RESULT();
}

int lb_latent_attention_plain(const void* q, const void* pages, void* out, const int* positions, const int* token_segment, const int* block_table,
                              int tokens, int num_heads, int latent, int rope, int page_size, int num_pages, int max_blocks, float scale, int window,
                              int dtype, int* status, cudaStream_t stream, const float* sink) {
    if (tokens == 0) return 0;
    if (latent < 1 || latent > lb::kLatentThreads * lb::kLatentMaxDimsPerThread || rope < 0) return -2;
    lb::LatentLayout layout{page_size, num_pages, max_blocks, latent, rope};
    const size_t shared = (3 * static_cast<size_t>(lb::kLatentChunk) + 36 + latent + rope) * sizeof(float);
    if (shared > 48 * 1024) return -2;
    const dim3 grid(tokens, num_heads);
    LB_DISPATCH_DTYPE(dtype, {
        lb::latent_attention_plain_kernel<T><<<grid, lb::kLatentThreads, shared, stream>>>(
            static_cast<const T*>(q), static_cast<const T*>(pages), static_cast<T*>(out), positions, token_segment, block_table, layout, num_heads, scale,
            window, status, sink);
    })
    return LB_LAUNCH_RESULT();
}

// bfloat16; latent and rope multiples of 16, page sizes that are multiples of 16.  items: [num_items][2] (first token row, count),
// each at most tokens_per_cta consecutive tokens of one request; heads_per_cta * tokens_per_cta <= 64.  partial: splits > 1 only,
// [tokens][heads][splits][latent + 2] floats.  Returns -2 for sizes it does not take.
int lb_latent_attention_mma(const void* q, const void* pages, void* out, float* partial, const int* items, int num_items, const int* positions,
                            const int* token_segment, const int* block_table, int tokens, int num_heads, int latent, int rope, int page_size,
                            int num_pages, int max_blocks, float scale, int window, int heads_per_cta, int tokens_per_cta, int splits, int* status,
                            cudaStream_t stream, const float* sink) {
    if (num_items == 0 || tokens == 0) return 0;
    if (latent < 16 || latent % 16 != 0 || rope % 16 != 0 || page_size % 16 != 0 || heads_per_cta < 1 || tokens_per_cta < 1 ||
        heads_per_cta * tokens_per_cta > lb::kLatentMmaRows || splits < 1 || (splits > 1 && partial == nullptr))
        return -2;
    const int full = latent + rope;
    const size_t shared = static_cast<size_t>(3) * lb::kLatentMmaRows * (full + 8) * sizeof(__nv_bfloat16);
    if (shared > 227 * 1024) return -2;
    static lb::OncePerDevice once_narrow, once_wide;
    const bool wide = latent > 128;   // 256 channels of the sums per CTA: twice the accumulators, the scores computed half as often
    const cudaError_t allowed = wide ? lb::allow_shared_memory(once_wide, lb::latent_attention_mma_kernel<256>, 227 * 1024)
                                     : lb::allow_shared_memory(once_narrow, lb::latent_attention_mma_kernel<128>, 227 * 1024);
    if (allowed != cudaSuccess) return static_cast<int>(allowed);
    lb::LatentMmaParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.pages = static_cast<const __nv_bfloat16*>(pages);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.partial = partial;
    p.items = items;
    p.positions = positions;
    p.token_segment = token_segment;
    p.block_table = block_table;
    p.layout = lb::LatentLayout{page_size, num_pages, max_blocks, latent, rope};
    p.num_heads = num_heads;
    p.heads_per_cta = heads_per_cta;
    p.tokens_per_cta = tokens_per_cta;
    p.head_blocks = (num_heads + heads_per_cta - 1) / heads_per_cta;
    p.splits = splits;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    p.sink = sink;
    const int chunk = wide ? 256 : 128;
    const dim3 grid(num_items, p.head_blocks * splits, (latent + chunk - 1) / chunk);
    if (wide) {
        lb::latent_attention_mma_kernel<256><<<grid, lb::kLatentMmaThreads, shared, stream>>>(p);
    } else {
        lb::latent_attention_mma_kernel<128><<<grid, lb::kLatentMmaThreads, shared, stream>>>(p);
    }
    if (splits > 1) lb::latent_merge_kernel<<<tokens * num_heads, 128, splits * sizeof(float), stream>>>(partial, static_cast<__nv_bfloat16*>(out), splits, latent, sink, num_heads);
    return LB_LAUNCH_RESULT();
}

// a [tokens][heads][k], out [tokens][heads][n] and gate (or null) addressed by (token stride, head stride) in elements; b [heads][k][n]
// if b_is_kn, else [heads][n][k].  bfloat16; k and n multiples of 16; every row 16-byte aligned (gate: 4-byte).  -2 otherwise.
int lb_heads_product(const void* a, long long a_token_stride, int a_head_stride, const void* b, int b_is_kn, void* out, long long out_token_stride,
                     int out_head_stride, const void* gate, long long gate_token_stride, int gate_head_stride, int tokens, int heads, int k, int n,
                     cudaStream_t stream) {
    if (tokens == 0 || heads == 0) return 0;
    if (k < 16 || n < 16 || k % 16 != 0 || n % 16 != 0 || a_token_stride % 8 != 0 || a_head_stride % 8 != 0 || out_token_stride % 2 != 0 ||
        out_head_stride % 2 != 0 || (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 4 != 0 ||
        (gate != nullptr && (gate_token_stride % 2 != 0 || gate_head_stride % 2 != 0 || reinterpret_cast<uintptr_t>(gate) % 4 != 0)))
        return -2;
    // blocks of 64 columns are shared out over grid.z as far as that is needed to fill the GPU, and to fit a CTA's share into shared memory
    const int token_blocks = (tokens + 63) / 64, column_blocks = (n + 63) / 64;
    int shares = (2 * lb::multiprocessor_count() + token_blocks * heads - 1) / (token_blocks * heads);
    shares = shares < 1 ? 1 : (shares > column_blocks ? column_blocks : shares);
    int blocks_per_cta = (column_blocks + shares - 1) / shares;
    auto shared_bytes = [&](int blocks) {
        return (static_cast<size_t>(64) * (k + 8) + (b_is_kn ? static_cast<size_t>(k) * (blocks * 64 + 8) : static_cast<size_t>(blocks) * 64 * (k + 8))) * sizeof(__nv_bfloat16);
    };
    while (blocks_per_cta > 1 && shared_bytes(blocks_per_cta) > 100 * 1024) --blocks_per_cta;   // two CTAs an SM at least
    const size_t shared = shared_bytes(blocks_per_cta);
    if (shared > 227 * 1024) return -2;
    static lb::OncePerDevice once_kn, once_nk;
    const cudaError_t allowed = b_is_kn ? lb::allow_shared_memory(once_kn, lb::heads_product_kernel<true>, 227 * 1024)
                                        : lb::allow_shared_memory(once_nk, lb::heads_product_kernel<false>, 227 * 1024);
    if (allowed != cudaSuccess) return static_cast<int>(allowed);
    lb::HeadsProductParams p;
    p.a = static_cast<const __nv_bfloat16*>(a);
    p.a_token_stride = a_token_stride;
    p.a_head_stride = a_head_stride;
    p.b = static_cast<const __nv_bfloat16*>(b);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.out_token_stride = out_token_stride;
    p.out_head_stride = out_head_stride;
    p.gate = static_cast<const __nv_bfloat16*>(gate);
    p.gate_token_stride = gate_token_stride;
    p.gate_head_stride = gate_head_stride;
    p.tokens = tokens;
    p.k = k;
    p.n = n;
    p.blocks_per_cta = blocks_per_cta;
    const dim3 grid(token_blocks, heads, (column_blocks + blocks_per_cta - 1) / blocks_per_cta);
    if (b_is_kn) lb::heads_product_kernel<true><<<grid, 128, shared, stream>>>(p);
    else lb::heads_product_kernel<false><<<grid, 128, shared, stream>>>(p);
    return LB_LAUNCH_RESULT();
}

int lb_gate_heads(const void* values, const void* gate, int gate_stride, void* out, int tokens, int num_heads, int value_dim, int dtype,
                  cudaStream_t stream) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::gate_heads_kernel<T><<<tokens, 256, 0, stream>>>(static_cast<const T*>(values), static_cast<const T*>(gate), gate_stride, static_cast<T*>(out),
                                                              tokens, num_heads, value_dim);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
