// Split-K flash-decode grouped-query attention over the paged KV cache.
//
// Work item = (query row, KV head): the G = heads / kv_heads query heads that share a KV head are processed
// together, so every K/V byte is read once per item.  The key range of an item is cut into splits of
// `pages_per_split` pages (grid.y); each CTA produces a partial (max, sum, accumulator) triple per head in the
// caller's scratch buffer and a second small kernel merges the splits.  The work is KV streaming (HBM-bound).
// Chunks of several positions per sequence (prefill) put 16 / G consecutive positions into one item of the fast path:
// the 16 fragment rows of the tensor-core products are positions x heads, each row with its own causal key count,
// so the K/V bytes of a sequence are streamed 16 / G times less often than with one item per position.
//
// Fast path (bf16 pools, 64-token pages, head_dim 64 or 128): a producer warp stages K and V pages with
// non-multicast TMA (cp.async.bulk.tensor, 128-byte swizzle) through a ring of shared-memory stages guarded by
// mbarriers; eight consumer warps in two groups (a group per page, 16 tokens per warp) compute Q.K^T and P.V with bf16 mma.sync
// (m16n8k16, f32 accumulation, fragments fetched with ldmatrix from the swizzled tiles), keep an online softmax
// per row, reduce row maxima and sums with quad shuffles and merge through shared memory.
//
// Generic path (f32 pools, other head sizes or page sizes): one (row, head) per CTA with plain loads and f32
// FMAs -- this is the path the f32 parity configuration runs on.
//
// Reference semantics: src/ops/attention.cpp:65-95 (scores * f32(1/sqrt(hd)), softmax, P.V) with the causal rule
// key_pos <= query_pos (src/ops/attention.cpp:52-57) expressed as a per-row key count.
#include "common.cuh"
#include "kv_cache.cuh"

#include <cmath>
#include <mutex>

namespace b200 {
namespace {

struct AttnParams {
    const float* q;    // [rows, heads, head_dim]
    int rows, tokens_per_sequence, heads, causal;
    int positions_per_item;   // tensor-core kernel: consecutive positions of one sequence that share a CTA (1 in decode)
    KvView kv;
    int pages_per_split, num_splits;
    int items;         // persistent tensor-core kernel: items the grid walks (grid x otherwise)
    float* part_o;     // [rows*heads, num_splits, head_dim]
    float* part_ml;    // [rows*heads, num_splits, 2]
    float* out;        // [rows, heads*head_dim]
    __nv_bfloat16 *out_hi, *out_lo;  // optional: result as a shadow (bf16 hi + lo planes) instead of `out`
    float scale;
    int32_t* status;
};

struct SplitPlan { int pages_total, pages_per_split, num_splits; };

SplitPlan plan_splits(int64_t rows, int kv_heads, int max_length, int page_size) {
    SplitPlan s{};
    s.pages_total = (max_length + page_size - 1) / page_size;
    if (s.pages_total < 1) s.pages_total = 1;
    const int64_t items = rows * kv_heads;
    // Enough CTAs to fill the SMs about three times (the scheduler evens out unequal items), but 8 to 16 pages
    // (128 to 512 KB of K and V) per CTA: a shorter stream is mostly pipeline ramp.
    const int64_t fill = 444;
    const int64_t want_splits = (fill + items - 1) / items;
    int64_t pps = s.pages_total / want_splits;
    if (pps < 8) pps = 8;
    if (pps > 16) pps = 16;
    if (items * ((s.pages_total + pps - 1) / pps) > 32768) pps = s.pages_total;
    // short contexts: one CTA per (row, KV head), no merge kernel - also up to 32 pages once the items alone give every SM a
    // CTA (a decode step is a chain of dependent launches: the merge launch costs more than the shorter streams save)
    if (s.pages_total <= 16 || (s.pages_total <= 32 && items >= 148)) pps = s.pages_total;
    if (pps > s.pages_total) pps = s.pages_total;
    s.pages_per_split = static_cast<int>(pps);
    s.num_splits = (s.pages_total + s.pages_per_split - 1) / s.pages_per_split;
    return s;
}

// Final attention value: f32, or the shadow planes when the caller asked for them.
__device__ __forceinline__ void store_result(const AttnParams& p, int64_t at, float value) {
    if (p.out_hi) {
        const __nv_bfloat16 hi = __float2bfloat16_rn(value);
        p.out_hi[at] = hi;
        p.out_lo[at] = __float2bfloat16_rn(value - __bfloat162float(hi));
    } else {
        p.out[at] = value;
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kConsumerWarps = 8;   // two groups of four: group g takes pages g, g+2, ... so two pages are in the
constexpr int kGroupWarps = 4;      // tensor-core pipeline at a time; a warp owns 16 tokens of its group's page
constexpr int kFastThreads = (kConsumerWarps + 1) * 32;
constexpr int kHalfTileBytes = 64 * 128;  // one TMA box: 64 tokens x 64 bf16
constexpr int kFastControlBytes = 256;    // behind the ring: full / empty barriers (at most 128 bytes), the give-up flag at 192

template <int HD, int STAGES> struct FastShape {
    static constexpr int halves = HD / 64;
    static constexpr int tile_bytes = halves * kHalfTileBytes;  // K or V page
    static constexpr int stage_bytes = 2 * tile_bytes;
    static constexpr int stages = STAGES;  // 6 x 32 KB (head_dim 128) or 8 / 6 x 16 KB (head_dim 64) of K and V in flight per CTA
    static constexpr int smem_bytes = stages * stage_bytes + 1024 + kFastControlBytes;   // 1024: slack of the 1024-byte alignment
};

// Byte offset of 16-byte chunk `chunk` (8 features) of token `token` inside a swizzled K or V page.
__device__ __forceinline__ uint32_t tile_offset(int token, int chunk) {
    return static_cast<uint32_t>((chunk >> 3) * kHalfTileBytes + token * 128 + (((chunk & 7) ^ (token & 7)) << 4));
}

// Barrier over the consumer warps only (the producer warp keeps streaming).
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

// Pages per split for a sequence of `pages` cached pages: the splits the sequence needs at the planned size share its
// pages evenly (17 pages planned as 16 + 1 become 9 + 8).
__device__ __forceinline__ int balanced_pages_per_split(int pages, int planned) {
    const int needed = (pages + planned - 1) / planned;
    return needed > 0 ? (pages + needed - 1) / needed : planned;
}

// MULTI: items of several positions (prefill chunks); the decode instantiation keeps one position per item and one key
// count for all of its rows.
template <int HD, int STAGES, bool MULTI>
__global__ void __launch_bounds__(kFastThreads) attention_mma_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                     const __grid_constant__ CUtensorMap vmap,
                                                                     const AttnParams p) {
    using S = FastShape<HD, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::stages * S::stage_bytes);
    uint64_t* empty = full + S::stages;

    grid_dependency_wait();   // q, the cache and the lengths come from the preceding kernels
    grid_launch_dependents();
    // An item is (sequence, block of consecutive positions, KV head).  The 16 fragment rows of a warp hold the block's
    // positions times the head group: row r = position r / group, query head r % group.  Decode: one position, rows =
    // the group.  Prefill: 16 / group positions share every K/V byte the CTA streams.
    const int item = blockIdx.x, split = blockIdx.y;
    const int kvh = item % p.kv.kv_heads, block = item / p.kv.kv_heads;
    const int positions = MULTI ? p.positions_per_item : 1;
    const int blocks_per_sequence = (p.tokens_per_sequence + positions - 1) / positions;
    const int sequence = block / blocks_per_sequence;
    const int t_first = (block - sequence * blocks_per_sequence) * positions;
    const int t_count = MULTI ? min(positions, p.tokens_per_sequence - t_first) : 1;
    const int row = sequence * p.tokens_per_sequence + t_first;   // first activation row of the item
    const int base_len = p.kv.lengths[sequence];
    const int kv_len = base_len + (p.causal ? t_first + t_count : 0);   // keys the item's last position sees
    int page_end = (kv_len + kFastPageSize - 1) / kFastPageSize;
    const int per_split = balanced_pages_per_split(page_end, p.pages_per_split);
    const int page_begin = split * per_split;
    if (page_end > page_begin + per_split) page_end = page_begin + per_split;
    if (page_begin >= page_end) return;  // uniform for the CTA
    const int pages = page_end - page_begin;
    const int group = p.heads / p.kv.kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kGroupWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();

    float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    if (warp == kConsumerWarps) {
        // ---- producer: all lanes walk the loop together, lane 0 waits and issues ----
        if (lane == 0) { tma_prefetch_descriptor(&kmap); tma_prefetch_descriptor(&vmap); }
        const int32_t* table = p.kv.page_table + static_cast<int64_t>(sequence) * p.kv.pages_per_seq + page_begin;
        bool alive = true;
        for (int i = 0; i < pages && alive; ++i) {
            if (lane == 0) {
                const int s = i % S::stages;
                const uint32_t phase = (i / S::stages) & 1;
                if (!mbar_wait(&empty[s], phase ^ 1)) {
                    atomicExch(p.status, B200_DEVICE_TIMEOUT);
                    alive = false;
                } else {
                    const int page = table[i];
                    const int y = (page * p.kv.kv_heads + kvh) * kFastPageSize;
                    uint8_t* kdst = smem + s * S::stage_bytes;
                    uint8_t* vdst = kdst + S::tile_bytes;
                    mbar_expect_tx(&full[s], S::stage_bytes);
#pragma unroll
                    for (int h = 0; h < S::halves; ++h) {
                        tma_load_2d(kdst + h * kHalfTileBytes, &kmap, h * 64, y, &full[s]);
                        tma_load_2d(vdst + h * kHalfTileBytes, &vmap, h * 64, y, &full[s]);
                    }
                }
            }
            alive = __shfl_sync(0xffffffffu, alive, 0);
        }
    } else {
        // ---- consumers ----
        const int g = lane >> 2, t = lane & 3;
        uint32_t qa[HD / 16][4];
        // this thread's two fragment rows: position and head inside the item, and the keys each may see
        const int pos0 = MULTI ? g / group : 0, pos1 = MULTI ? (g + 8) / group : 0;
        const bool v0 = g < group * t_count, v1 = g + 8 < group * t_count;
        const int limit0 = MULTI ? (v0 ? base_len + (p.causal ? t_first + pos0 + 1 : 0) : 0) : kv_len;
        const int limit1 = MULTI ? (v1 ? base_len + (p.causal ? t_first + pos1 + 1 : 0) : 0) : kv_len;
        {
            const float* q0 = p.q + (static_cast<int64_t>(row + pos0) * p.heads + kvh * group + (g - pos0 * group)) * HD;
            const float* q1 = p.q + (static_cast<int64_t>(row + pos1) * p.heads + kvh * group + (g + 8 - pos1 * group)) * HD;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const int c = kk * 16 + 2 * t;
                qa[kk][0] = v0 ? pack_bf16(q0[c], q0[c + 1]) : 0u;
                qa[kk][1] = v1 ? pack_bf16(q1[c], q1[c + 1]) : 0u;
                qa[kk][2] = v0 ? pack_bf16(q0[c + 8], q0[c + 9]) : 0u;
                qa[kk][3] = v1 ? pack_bf16(q1[c + 8], q1[c + 9]) : 0u;
            }
        }
        const int tok0 = (warp & (kGroupWarps - 1)) * 16;
        const int group_index = warp / kGroupWarps;
        const int mi = lane >> 3, ri = lane & 7;
        bool alive = true;
        for (int i = group_index; i < pages && alive; i += kConsumerWarps / kGroupWarps) {
            const int s = i % S::stages;
            const uint32_t phase = (i / S::stages) & 1;
            if (!mbar_wait(&full[s], phase)) {
                if (lane == 0) atomicExch(p.status, B200_DEVICE_TIMEOUT);
                alive = false;
                break;
            }
            const uint32_t kbase = smem_u32(smem + s * S::stage_bytes);
            const uint32_t vbase = kbase + S::tile_bytes;

            float sc[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t r[4];
                ldmatrix_x4(r, kbase + tile_offset(tok0 + (mi >> 1) * 8 + ri, 2 * kk + (mi & 1)));
                mma_bf16(sc[0], qa[kk], r[0], r[1]);
                mma_bf16(sc[1], qa[kk], r[2], r[3]);
            }
            // scale, mask keys at or beyond the row's key count, online softmax per row (g and g+8)
            const int token_base = (page_begin + i) * kFastPageSize + tok0 + 2 * t;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int token = token_base + n * 8 + (e & 1);
                    const float v = token < (MULTI ? ((e >> 1) ? limit1 : limit0) : kv_len) ? sc[n][e] * p.scale : -INFINITY;
                    sc[n][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float corr[2], safe[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_row[h], mx[h]);
                safe[h] = m_new == -INFINITY ? 0.0f : m_new;
                corr[h] = expf(m_row[h] - safe[h]);
                m_row[h] = m_new;
            }
            float sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sc[n][e] = expf(sc[n][e] - safe[e >> 1]);
                    sum[e >> 1] += sc[n][e];
                }
            l_row[0] = l_row[0] * corr[0] + sum[0];
            l_row[1] = l_row[1] * corr[1] + sum[1];
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            uint32_t pa[4];
            pa[0] = pack_bf16(sc[0][0], sc[0][1]);
            pa[1] = pack_bf16(sc[0][2], sc[0][3]);
            pa[2] = pack_bf16(sc[1][0], sc[1][1]);
            pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
            for (int j = 0; j < HD / 8; j += 2) {
                uint32_t r[4];
                ldmatrix_x4_trans(r, vbase + tile_offset(tok0 + (mi & 1) * 8 + ri, j + (mi >> 1)));
                mma_bf16(o[j], pa, r[0], r[1]);
                mma_bf16(o[j + 1], pa, r[2], r[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 1);
            l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 2);
        }
    }
    __syncthreads();  // every page has been consumed: the stage memory can be reused for the merge

    float* merge_o = reinterpret_cast<float*>(smem);                       // [warps][group][HD]
    float* merge_ml = merge_o + kConsumerWarps * 16 * HD;                   // [warps][16][2]
    if (warp < kConsumerWarps) {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = g + 8 * h;
            if (r < group * t_count) {
                float* dst = merge_o + (warp * 16 + r) * HD + 2 * t;
#pragma unroll
                for (int j = 0; j < HD / 8; ++j) {
                    dst[j * 8] = o[j][2 * h];
                    dst[j * 8 + 1] = o[j][2 * h + 1];
                }
                if (t == 0) {
                    merge_ml[(warp * 16 + r) * 2] = m_row[h];
                    merge_ml[(warp * 16 + r) * 2 + 1] = l_row[h];
                }
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * t_count * HD; i += kFastThreads) {
        const int r = i / HD, d = i - r * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) m = fmaxf(m, merge_ml[(w * 16 + r) * 2]);
        float acc = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
            const float mw = merge_ml[(w * 16 + r) * 2];
            const float weight = mw == -INFINITY ? 0.0f : expf(mw - m);
            acc += weight * merge_o[(w * 16 + r) * HD + d];
            l += weight * merge_ml[(w * 16 + r) * 2 + 1];
        }
        const int position = MULTI ? r / group : 0;
        const int64_t head_item = static_cast<int64_t>(row + position) * p.heads + kvh * group + (r - position * group);
        if (p.num_splits == 1) {
            store_result(p, head_item * HD + d, acc / l);
        } else {
            p.part_o[(head_item * p.num_splits + split) * HD + d] = acc;
            if (d == 0) {
                p.part_ml[(head_item * p.num_splits + split) * 2] = m;
                p.part_ml[(head_item * p.num_splits + split) * 2 + 1] = l;
            }
        }
    }
}

// The same kernel for decode with more units of work (item, split of its pages) than resident CTAs: a CTA walks the units
// blockIdx.x, + gridDim.x, ... and its
// producer warp runs ahead into the next item's pages while the consumers finish the current one, so the K/V stream of an
// SM does not stop at item boundaries (an item of 17 pages is ~290 KB: a sixth of its time was pipeline ramp).  The
// cross-warp merge then has its own shared memory behind the ring instead of re-using drained stages.
template <int HD, int STAGES>
__global__ void __launch_bounds__(kFastThreads) attention_persistent_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                     const __grid_constant__ CUtensorMap vmap,
                                                                     const AttnParams p) {
    using S = FastShape<HD, STAGES>;
    constexpr bool MULTI = false, PERSIST = true;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::stages * S::stage_bytes);
    uint64_t* empty = full + S::stages;
    volatile int* gave_up = reinterpret_cast<volatile int*>(smem + S::stages * S::stage_bytes + 192);   // a consumer's wait ran out

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    grid_dependency_wait();   // q, the cache and the lengths come from the preceding kernels
    grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < S::stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kGroupWarps);
        }
        *gave_up = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // An item is (sequence, block of consecutive positions, KV head).  The 16 fragment rows of a warp hold the block's
    // positions times the head group: row r = position r / group, query head r % group.  Decode: one position, rows =
    // the group.  Prefill: 16 / group positions share every K/V byte the CTA streams.
    const int group = p.heads / p.kv.kv_heads;
    const int positions = MULTI ? p.positions_per_item : 1;
    const int blocks_per_sequence = (p.tokens_per_sequence + positions - 1) / positions;
    // units of work: (item, split of its pages); without PERSIST the grid has one CTA per unit
    const int units = PERSIST ? p.items * p.num_splits : static_cast<int>(blockIdx.x) + 1;
    // the cross-warp merge: [warps][16][HD] partial outputs and [warps][16][2] (max, sum); PERSIST keeps only the rows of a
    // decode item ([warps][group][...]) in its own memory behind the barriers
    float* merge_o = PERSIST ? reinterpret_cast<float*>(smem + S::stages * S::stage_bytes + kFastControlBytes) : reinterpret_cast<float*>(smem);
    const int merge_rows = PERSIST ? group : 16;
    float* merge_ml = merge_o + kConsumerWarps * merge_rows * HD;
    int walked = 0;   // pages this CTA has been through before the current item: stage and phase follow from it

    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        const int item = PERSIST ? unit / p.num_splits : unit;
        const int split = PERSIST ? unit - item * p.num_splits : static_cast<int>(blockIdx.y);
        const int kvh = item % p.kv.kv_heads, block = item / p.kv.kv_heads;
        const int sequence = block / blocks_per_sequence;
        const int t_first = (block - sequence * blocks_per_sequence) * positions;
        const int t_count = MULTI ? min(positions, p.tokens_per_sequence - t_first) : 1;
        const int row = sequence * p.tokens_per_sequence + t_first;   // first activation row of the item
        const int base_len = p.kv.lengths[sequence];
        const int kv_len = base_len + (p.causal ? t_first + t_count : 0);   // keys the item's last position sees
        int page_end = (kv_len + kFastPageSize - 1) / kFastPageSize;
        const int per_split = balanced_pages_per_split(page_end, p.pages_per_split);
        const int page_begin = split * per_split;
        if (page_end > page_begin + per_split) page_end = page_begin + per_split;
        if (page_begin >= page_end) continue;  // uniform for the CTA (a sequence without keys writes nothing, as before)
        const int pages = page_end - page_begin;

        if (warp == kConsumerWarps) {
            // ---- producer: all lanes walk the loop together, lane 0 waits and issues ----
            if (lane == 0 && walked == 0) { tma_prefetch_descriptor(&kmap); tma_prefetch_descriptor(&vmap); }
            const int32_t* table = p.kv.page_table + static_cast<int64_t>(sequence) * p.kv.pages_per_seq + page_begin;
            bool alive = true;
            for (int i = 0; i < pages && alive; ++i) {
                if (lane == 0) {
                    const int n = walked + i;
                    const int s = n % S::stages;
                    const uint32_t phase = (n / S::stages) & 1;
                    if (!mbar_wait(&empty[s], phase ^ 1)) {
                        atomicExch(p.status, B200_DEVICE_TIMEOUT);
                        alive = false;
                    } else {
                        const int page = table[i];
                        const int y = (page * p.kv.kv_heads + kvh) * kFastPageSize;
                        uint8_t* kdst = smem + s * S::stage_bytes;
                        uint8_t* vdst = kdst + S::tile_bytes;
                        mbar_expect_tx(&full[s], S::stage_bytes);
#pragma unroll
                        for (int h = 0; h < S::halves; ++h) {
                            tma_load_2d(kdst + h * kHalfTileBytes, &kmap, h * 64, y, &full[s]);
                            tma_load_2d(vdst + h * kHalfTileBytes, &vmap, h * 64, y, &full[s]);
                        }
                    }
                }
                alive = __shfl_sync(0xffffffffu, alive, 0);
            }
            walked += pages;
            if (!alive) break;   // the consumers run into their own bounded waits
            continue;
        }

        // ---- consumers ----
        float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.0f, 0.0f};
        float o[HD / 8][4];
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
        const int g = lane >> 2, t = lane & 3;
        uint32_t qa[HD / 16][4];
        // this thread's two fragment rows: position and head inside the item, and the keys each may see
        const int pos0 = MULTI ? g / group : 0, pos1 = MULTI ? (g + 8) / group : 0;
        const bool v0 = g < group * t_count, v1 = g + 8 < group * t_count;
        const int limit0 = MULTI ? (v0 ? base_len + (p.causal ? t_first + pos0 + 1 : 0) : 0) : kv_len;
        const int limit1 = MULTI ? (v1 ? base_len + (p.causal ? t_first + pos1 + 1 : 0) : 0) : kv_len;
        {
            const float* q0 = p.q + (static_cast<int64_t>(row + pos0) * p.heads + kvh * group + (g - pos0 * group)) * HD;
            const float* q1 = p.q + (static_cast<int64_t>(row + pos1) * p.heads + kvh * group + (g + 8 - pos1 * group)) * HD;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const int c = kk * 16 + 2 * t;
                qa[kk][0] = v0 ? pack_bf16(q0[c], q0[c + 1]) : 0u;
                qa[kk][1] = v1 ? pack_bf16(q1[c], q1[c + 1]) : 0u;
                qa[kk][2] = v0 ? pack_bf16(q0[c + 8], q0[c + 9]) : 0u;
                qa[kk][3] = v1 ? pack_bf16(q1[c + 8], q1[c + 9]) : 0u;
            }
        }
        const int tok0 = (warp & (kGroupWarps - 1)) * 16;
        const int group_index = warp / kGroupWarps;
        const int mi = lane >> 3, ri = lane & 7;
        bool alive = true;
        // the two warp groups alternate over the CTA's pages as a whole, not per item: stage n belongs to group n % 2
        for (int i = (group_index + walked) & 1; i < pages && alive; i += kConsumerWarps / kGroupWarps) {
            const int n = walked + i;
            const int s = n % S::stages;
            const uint32_t phase = (n / S::stages) & 1;
            if (!mbar_wait(&full[s], phase)) {
                if (lane == 0) { atomicExch(p.status, B200_DEVICE_TIMEOUT); *gave_up = 1; }
                alive = false;
                break;
            }
            const uint32_t kbase = smem_u32(smem + s * S::stage_bytes);
            const uint32_t vbase = kbase + S::tile_bytes;

            float sc[2][4];
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2) sc[n2][0] = sc[n2][1] = sc[n2][2] = sc[n2][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t r[4];
                ldmatrix_x4(r, kbase + tile_offset(tok0 + (mi >> 1) * 8 + ri, 2 * kk + (mi & 1)));
                mma_bf16(sc[0], qa[kk], r[0], r[1]);
                mma_bf16(sc[1], qa[kk], r[2], r[3]);
            }
            // scale, mask keys at or beyond the row's key count, online softmax per row (g and g+8)
            const int token_base = (page_begin + i) * kFastPageSize + tok0 + 2 * t;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int token = token_base + n2 * 8 + (e & 1);
                    const float v = token < (MULTI ? ((e >> 1) ? limit1 : limit0) : kv_len) ? sc[n2][e] * p.scale : -INFINITY;
                    sc[n2][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float corr[2], safe[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_row[h], mx[h]);
                safe[h] = m_new == -INFINITY ? 0.0f : m_new;
                corr[h] = expf(m_row[h] - safe[h]);
                m_row[h] = m_new;
            }
            float sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sc[n2][e] = expf(sc[n2][e] - safe[e >> 1]);
                    sum[e >> 1] += sc[n2][e];
                }
            l_row[0] = l_row[0] * corr[0] + sum[0];
            l_row[1] = l_row[1] * corr[1] + sum[1];
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            uint32_t pa[4];
            pa[0] = pack_bf16(sc[0][0], sc[0][1]);
            pa[1] = pack_bf16(sc[0][2], sc[0][3]);
            pa[2] = pack_bf16(sc[1][0], sc[1][1]);
            pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
            for (int j = 0; j < HD / 8; j += 2) {
                uint32_t r[4];
                ldmatrix_x4_trans(r, vbase + tile_offset(tok0 + (mi & 1) * 8 + ri, j + (mi >> 1)));
                mma_bf16(o[j], pa, r[0], r[1]);
                mma_bf16(o[j + 1], pa, r[2], r[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        walked += pages;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 1);
            l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 2);
        }
        // Every consumer warp is through its pages: without PERSIST the whole ring is drained and serves the merge; with it
        // the merge has its own memory, which the previous item's readers have left (second barrier below).
        consumer_barrier();
        if (*gave_up) break;   // the same for every consumer warp after the barrier: nobody is left waiting at the next one
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = g + 8 * h;
            if (r < group * t_count) {
                float* dst = merge_o + (warp * merge_rows + r) * HD + 2 * t;
#pragma unroll
                for (int j = 0; j < HD / 8; ++j) {
                    dst[j * 8] = o[j][2 * h];
                    dst[j * 8 + 1] = o[j][2 * h + 1];
                }
                if (t == 0) {
                    merge_ml[(warp * merge_rows + r) * 2] = m_row[h];
                    merge_ml[(warp * merge_rows + r) * 2 + 1] = l_row[h];
                }
            }
        }
        consumer_barrier();
        for (int i = threadIdx.x; i < group * t_count * HD; i += kConsumerWarps * 32) {
            const int r = i / HD, d = i - r * HD;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) m = fmaxf(m, merge_ml[(w * merge_rows + r) * 2]);
            float acc = 0.0f, l = 0.0f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float mw = merge_ml[(w * merge_rows + r) * 2];
                const float weight = mw == -INFINITY ? 0.0f : expf(mw - m);
                acc += weight * merge_o[(w * merge_rows + r) * HD + d];
                l += weight * merge_ml[(w * merge_rows + r) * 2 + 1];
            }
            const int position = MULTI ? r / group : 0;
            const int64_t head_item = static_cast<int64_t>(row + position) * p.heads + kvh * group + (r - position * group);
            if (p.num_splits == 1) {
                store_result(p, head_item * HD + d, acc / l);
            } else {
                p.part_o[(head_item * p.num_splits + split) * HD + d] = acc;
                if (d == 0) {
                    p.part_ml[(head_item * p.num_splits + split) * 2] = m;
                    p.part_ml[(head_item * p.num_splits + split) * 2 + 1] = l;
                }
            }
        }
    }
}

// Generic path: one (row, head) per CTA, four warps stride over the tokens of the split.
constexpr int kGenericThreads = 128;
constexpr int kMaxDimsPerLane = 8;  // head_dim <= 256

__global__ void __launch_bounds__(kGenericThreads) attention_generic_kernel(const AttnParams p) {
    __shared__ float merge_ml[4][2];
    extern __shared__ float merge_o[];  // [4][head_dim]
    grid_dependency_wait();
    grid_launch_dependents();
    const int hd = p.kv.head_dim;
    const int item = blockIdx.x, split = blockIdx.y;
    const int row = item / p.heads, head = item % p.heads;
    const int kvh = head / (p.heads / p.kv.kv_heads);
    const int sequence = row / p.tokens_per_sequence;
    const int kv_len = p.kv.lengths[sequence] + (p.causal ? row % p.tokens_per_sequence + 1 : 0);
    const int per_split = balanced_pages_per_split((kv_len + p.kv.page_size - 1) / p.kv.page_size, p.pages_per_split);
    const int begin = split * per_split * p.kv.page_size;
    int end = begin + per_split * p.kv.page_size;
    if (end > kv_len) end = kv_len;
    if (begin >= end) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* q = p.q + (static_cast<int64_t>(row) * p.heads + head) * hd;
    float qv[kMaxDimsPerLane], acc[kMaxDimsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < hd ? q[d] : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int token = begin + warp; token < end; token += 4) {
        const int64_t at = kv_offset(p.kv, sequence, token, kvh);
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < kMaxDimsPerLane; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) dot = fmaf(qv[i], kv_load(p.kv, 0, at + d), dot);
        }
        const float score = warp_sum(dot) * p.scale;
        const float m_new = fmaxf(m, score);
        const float corr = expf(m - m_new), weight = expf(score - m_new);
        l = l * corr + weight;
#pragma unroll
        for (int i = 0; i < kMaxDimsPerLane; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) acc[i] = fmaf(weight, kv_load(p.kv, 1, at + d), acc[i] * corr);
        }
        m = m_new;
    }
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) merge_o[warp * hd + d] = acc[i];
    }
    if (lane == 0) { merge_ml[warp][0] = m; merge_ml[warp][1] = l; }
    __syncthreads();
    const int64_t head_item = static_cast<int64_t>(row) * p.heads + head;
    for (int d = threadIdx.x; d < hd; d += kGenericThreads) {
        float mm = -INFINITY;
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge_ml[w][0]);
        float a = 0.0f, ll = 0.0f;
        for (int w = 0; w < 4; ++w) {
            const float weight = merge_ml[w][0] == -INFINITY ? 0.0f : expf(merge_ml[w][0] - mm);
            a += weight * merge_o[w * hd + d];
            ll += weight * merge_ml[w][1];
        }
        if (p.num_splits == 1) {
            store_result(p, head_item * hd + d, a / ll);
        } else {
            p.part_o[(head_item * p.num_splits + split) * hd + d] = a;
            if (d == 0) {
                p.part_ml[(head_item * p.num_splits + split) * 2] = mm;
                p.part_ml[(head_item * p.num_splits + split) * 2 + 1] = ll;
            }
        }
    }
}

// Merge of the split partials: one (row, head) per CTA.
__global__ void attention_combine_kernel(const AttnParams p) {
    grid_dependency_wait();
    grid_launch_dependents();
    const int hd = p.kv.head_dim;
    const int64_t head_item = blockIdx.x;
    const int row = static_cast<int>(head_item / p.heads);
    const int sequence = row / p.tokens_per_sequence;
    const int kv_len = p.kv.lengths[sequence] + (p.causal ? row % p.tokens_per_sequence + 1 : 0);
    const int pages = (kv_len + p.kv.page_size - 1) / p.kv.page_size;
    const int per_split = balanced_pages_per_split(pages, p.pages_per_split);
    int valid = (pages + per_split - 1) / per_split;   // splits whose CTA had pages and wrote a partial
    if (valid > p.num_splits) valid = p.num_splits;
    const float* ml = p.part_ml + head_item * p.num_splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < valid; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.0f;
    for (int s = 0; s < valid; ++s) l += expf(ml[2 * s] - m) * ml[2 * s + 1];
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < valid; ++s) acc += expf(ml[2 * s] - m) * p.part_o[(head_item * p.num_splits + s) * hd + d];
        store_result(p, head_item * hd + d, acc / l);
    }
}

template <int HD, int STAGES> int launch_fast(const b200_kv_cache* cache, AttnParams p, cudaStream_t stream) {
    using S = FastShape<HD, STAGES>;
    const int blocks_per_sequence = (p.tokens_per_sequence + p.positions_per_item - 1) / p.positions_per_item;
    const int items = (p.rows / p.tokens_per_sequence) * blocks_per_sequence * p.kv.kv_heads;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    // Decode with more units of work than the SMs hold at once: persistent CTAs that stream across unit boundaries.
    const int group = p.heads / p.kv.kv_heads;
    const int merge_bytes = kConsumerWarps * group * (HD + 2) * static_cast<int>(sizeof(float));
    const int persist_bytes = S::smem_bytes + merge_bytes;   // the merge area follows the control block
    // With split items the units are dealt out in turn, which only balances when the sequences are equally long (what
    // the cache's owner knows on the host); ragged split batches keep one CTA per unit and the hardware's scheduling.
    if (p.positions_per_item == 1 && persist_bytes <= 232448 && static_cast<int64_t>(items) * p.num_splits > sm_count(device)
        && (p.num_splits == 1 || cache->even_lengths)) {
        auto kernel = attention_persistent_kernel<HD, STAGES>;
        B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, persist_bytes));
        int per_sm = 0;   // CTAs of this kernel an SM holds at once, asked of the runtime (1 if it cannot say)
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kFastThreads, static_cast<size_t>(persist_bytes)) != cudaSuccess || per_sm < 1) {
            cudaGetLastError();
            per_sm = 1;
        }
        const int resident = per_sm * sm_count(device);
        p.items = items;
        if (items * p.num_splits <= resident) {   // every unit has a CTA of its own anyway
            return cuda_status(launch_dependent(kernel, dim3(static_cast<unsigned>(items * p.num_splits)), dim3(kFastThreads),
                                                static_cast<size_t>(persist_bytes), stream, *kv_tensor_map(cache, 0), *kv_tensor_map(cache, 1), p),
                               "attention_mma_kernel launch");
        }
        p.items = items;
        return cuda_status(launch_dependent(kernel, dim3(static_cast<unsigned>(resident)), dim3(kFastThreads), static_cast<size_t>(persist_bytes),
                                            stream, *kv_tensor_map(cache, 0), *kv_tensor_map(cache, 1), p), "attention_mma_kernel launch");
    }
    auto kernel = p.positions_per_item > 1 ? attention_mma_kernel<HD, STAGES, true> : attention_mma_kernel<HD, STAGES, false>;
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::smem_bytes));
    const dim3 grid(static_cast<unsigned>(items), p.num_splits);
    return cuda_status(launch_dependent(kernel, grid, dim3(kFastThreads), S::smem_bytes, stream, *kv_tensor_map(cache, 0),
                                        *kv_tensor_map(cache, 1), p), "attention_mma_kernel launch");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" size_t b200_attention_scratch_bytes(int64_t rows, int32_t heads, int32_t kv_heads, int32_t head_dim,
                                               int32_t max_length, int32_t page_size) {
    if (rows <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || max_length <= 0 || page_size <= 0) return 0;
    const SplitPlan s = plan_splits(rows, kv_heads, max_length, page_size);
    if (s.num_splits == 1) return 256;
    return static_cast<size_t>(rows) * heads * s.num_splits * (head_dim + 2) * sizeof(float) + 256;
}

namespace {
int attention_launch(const float* q, int64_t rows, int32_t tokens_per_sequence, int32_t heads, const b200_kv_cache* cache,
                     int32_t max_length, int32_t causal, void* scratch, size_t scratch_bytes, float* out, __nv_bfloat16* out_hi,
                     __nv_bfloat16* out_lo, void* stream) {
    if (!q || !cache || (!out && !(out_hi && out_lo)) || rows <= 0 || tokens_per_sequence <= 0 || heads <= 0 || heads % cache->kv_heads
        || rows != static_cast<int64_t>(cache->sequences) * tokens_per_sequence || max_length <= 0) {
        set_error("b200_attention_decode: bad pointer, size or head grouping");
        return B200_BAD_ARGUMENT;
    }
    if (cache->head_dim > 32 * kMaxDimsPerLane) { set_error("b200_attention_decode: head_dim above 256 is not supported"); return B200_UNSUPPORTED; }
    {   // the kernels run on the current device: it must be the one that holds the cache (and, for the static entry, the scratch)
        int current = -1;
        B200_CUDA(cudaGetDevice(&current));
        if (current != cache->device) {
            set_error("b200_attention_decode: the cache lives on device %d, the current device is %d", cache->device, current);
            return B200_BAD_ARGUMENT;
        }
    }
    if (max_length > cache->capacity) max_length = cache->capacity;
    const int group = heads / cache->kv_heads;
    const bool fast = kv_tensor_map(cache, 0) && group <= 16 && (cache->head_dim == 64 || cache->head_dim == 128);
    // Chunks of several positions (prefill) on the tensor-core kernel: 16 / group consecutive positions share a CTA and one
    // CTA walks all pages of its item (the split sizes of the merge kernel are per row, the items' are per block).
    const int positions = fast && tokens_per_sequence > 1 ? (16 / group > 0 ? 16 / group : 1) : 1;
    SplitPlan plan = plan_splits(rows, cache->kv_heads, max_length, cache->page_size);
    if (positions > 1) {
        plan.pages_per_split = plan.pages_total;
        plan.num_splits = 1;
    }
    const size_t need = b200_attention_scratch_bytes(rows, heads, cache->kv_heads, cache->head_dim, max_length, cache->page_size);
    if (plan.num_splits > 1 && (!scratch || scratch_bytes < need)) {
        set_error("b200_attention_decode: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
        return B200_BAD_ARGUMENT;
    }
    AttnParams p{};
    p.q = q; p.rows = static_cast<int>(rows); p.tokens_per_sequence = tokens_per_sequence; p.heads = heads; p.causal = causal;
    p.positions_per_item = positions;
    p.kv = kv_view(cache);
    p.pages_per_split = plan.pages_per_split; p.num_splits = plan.num_splits;
    p.part_o = static_cast<float*>(scratch);
    p.part_ml = p.part_o ? p.part_o + static_cast<size_t>(rows) * heads * plan.num_splits * cache->head_dim : nullptr;
    p.out = out; p.out_hi = out_hi; p.out_lo = out_lo;
    p.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(cache->head_dim)));
    p.status = device_status_word(cache->device);
    if (!p.status) { set_error("b200_attention_decode: the device status word could not be allocated"); return B200_NO_DEVICE; }
    cudaStream_t s = as_stream(stream);
    int status;
    if (fast) {
        // head_dim 64 with more CTAs than SMs: a 96 KB ring lets two CTAs share an SM, so one CTA's pipeline ramp and
        // drain overlap the other's streaming; with fewer CTAs each keeps the deeper ring to itself.
        int device = 0;
        B200_CUDA(cudaGetDevice(&device));
        const int64_t ctas = (static_cast<int64_t>(p.rows) / tokens_per_sequence) * ((tokens_per_sequence + positions - 1) / positions)
                             * p.kv.kv_heads * p.num_splits;
        if (cache->head_dim == 128) status = launch_fast<128, 6>(cache, p, s);
        else if (ctas > sm_count(device)) status = launch_fast<64, 6>(cache, p, s);
        else status = launch_fast<64, 8>(cache, p, s);
    } else {
        const dim3 grid(static_cast<unsigned>(rows) * heads, plan.num_splits);
        status = cuda_status(launch_dependent(attention_generic_kernel, grid, dim3(kGenericThreads), sizeof(float) * 4 * cache->head_dim, s, p),
                             "attention_generic_kernel launch");
    }
    if (status != B200_OK || plan.num_splits == 1) return status;
    return cuda_status(launch_dependent(attention_combine_kernel, dim3(static_cast<unsigned>(rows) * heads), dim3(128), 0, s, p),
                       "attention_combine_kernel launch");
}
}  // namespace

extern "C" int b200_attention_decode(const float* q, int64_t rows, int32_t tokens_per_sequence, int32_t heads,
                                     const b200_kv_cache* cache, int32_t max_length, int32_t causal, void* scratch,
                                     size_t scratch_bytes, float* out, void* stream) {
    if (!out) { set_error("b200_attention_decode: bad pointer, size or head grouping"); return B200_BAD_ARGUMENT; }
    return attention_launch(q, rows, tokens_per_sequence, heads, cache, max_length, causal, scratch, scratch_bytes, out, nullptr, nullptr, stream);
}

extern "C" int b200_attention_decode_shadow(const float* q, int64_t rows, int32_t tokens_per_sequence, int32_t heads,
                                            const b200_kv_cache* cache, int32_t max_length, int32_t causal, void* scratch,
                                            size_t scratch_bytes, void* out_hi, void* out_lo, void* stream) {
    if (!out_hi || !out_lo) { set_error("b200_attention_decode_shadow: shadow planes missing"); return B200_BAD_ARGUMENT; }
    return attention_launch(q, rows, tokens_per_sequence, heads, cache, max_length, causal, scratch, scratch_bytes, nullptr,
                            static_cast<__nv_bfloat16*>(out_hi), static_cast<__nv_bfloat16*>(out_lo), stream);
}

// ---- allocation-free variant ------------------------------------------------------------------------------
// Split partials live in this fixed array of the library image instead of a caller workspace.  In host code the
// name below is only a handle for the runtime: the device address comes from cudaGetSymbolAddress, looked up once
// per device with that device current, and that address is what the kernels receive.
static __device__ __align__(256) unsigned char attention_static_scratch[B200_STATIC_SCRATCH_BYTES];

namespace {
std::mutex static_scratch_mutex;
void* static_scratch_address[64];

int static_scratch_for(int device, void** address) {
    std::lock_guard<std::mutex> lock(static_scratch_mutex);
    if (device < 0 || device >= 64) { set_error("b200_attention_decode_static: device %d out of range", device); return B200_BAD_ARGUMENT; }
    if (!static_scratch_address[device]) {
        int current = -1;
        B200_CUDA(cudaGetDevice(&current));
        if (current != device) B200_CUDA(cudaSetDevice(device));
        void* found = nullptr;
        const cudaError_t status = cudaGetSymbolAddress(&found, attention_static_scratch);
        if (current != device) cudaSetDevice(current);
        if (status != cudaSuccess || !found) return cuda_status(status == cudaSuccess ? cudaErrorInvalidSymbol : status,
                                                                "cudaGetSymbolAddress(attention_static_scratch)");
        static_scratch_address[device] = found;
    }
    *address = static_scratch_address[device];
    return B200_OK;
}
}  // namespace

extern "C" int b200_attention_decode_static(const float* q, int64_t rows, int32_t tokens_per_sequence, int32_t heads,
                                            const b200_kv_cache* cache, int32_t max_length, int32_t causal, float* out,
                                            void* stream) {
    if (!cache || rows <= 0 || heads <= 0 || max_length <= 0) {
        set_error("b200_attention_decode_static: bad pointer or size");
        return B200_BAD_ARGUMENT;
    }
    const int32_t bounded = max_length > cache->capacity ? cache->capacity : max_length;
    const size_t need = b200_attention_scratch_bytes(rows, heads, cache->kv_heads, cache->head_dim, bounded, cache->page_size);
    if (need > B200_STATIC_SCRATCH_BYTES) {
        set_error("b200_attention_decode_static: this shape needs %zu bytes of split partials, the built-in array holds %u; "
                  "call b200_attention_decode with a workspace of your own", need, static_cast<unsigned>(B200_STATIC_SCRATCH_BYTES));
        return B200_BAD_ARGUMENT;
    }
    if (!device_status_word_if_allocated(cache->device)) {
        set_error("b200_attention_decode_static: no status word on device %d (create the KV cache through b200_kv_cache_create)", cache->device);
        return B200_BAD_ARGUMENT;
    }
    void* scratch = nullptr;
    const int status = static_scratch_for(cache->device, &scratch);
    if (status != B200_OK) return status;
    return b200_attention_decode(q, rows, tokens_per_sequence, heads, cache, max_length, causal, scratch,
                                 B200_STATIC_SCRATCH_BYTES, out, stream);
}
