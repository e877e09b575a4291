// Dense projection for decode batches (up to 256 activation rows in token tiles of 128): y = epilogue(scale_rows(x @ W^T))
// with the WEIGHTS as the streamed operand.  A decode step reads every weight once and the activations are small, so the
// kernel is built to keep the weight stream going and to spend no tensor time on padding:
//
//   * operands are swapped against the prefill kernel (linear_gemm.cu): a 128-feature weight tile is the A operand
//     (M = 128) and the tokens are the N side of tcgen05.mma (N = rows of the token tile rounded up to 16).  A product
//     costs about max(51, N / 2) cycles when it re-uses the A operand of its predecessor (the hi and lo planes of the
//     activations are multiplied back to back against the same weight slice), so 32 rows cost less than half of what a
//     128-row token tile costs; up to 128 rows one CTA covers all tokens and every weight byte crosses L2 -> SM once;
//   * a CTA multiplies `tiles` (1, 2 or 4) adjacent weight tiles against each activation K block, one f32 accumulator
//     [128 features x N tokens] per tile in tensor memory, which divides the activation bytes pulled per weight byte;
//   * few feature tiles: K is split over a thread-block cluster (grid z, up to 8 CTAs); the partial accumulators are pushed
//     into the shared memory of the CTA that finishes the token row and summed there in a fixed order (results do not
//     depend on timing);
//   * warp 0 is the TMA producer (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast): the weight boxes of the
//     first ring fill are requested BEFORE griddepcontrol.wait (weights are constants), the activation boxes after it;
//     warp 1 owns tensor memory and issues the products; both warps walk their loops as whole warps in uniform control
//     flow, with ONE elected lane issuing a K block's instructions from fully unrolled code (tile count and plane count
//     are template parameters): issued from a loop with run-time bounds the same products took three times as long;
//   * all twelve warps read the accumulators back (tcgen05.ld: one feature per thread, 32 tokens per instruction; three
//     warps share a lane quarter) and write them transposed into row-major [token][feature] slabs, from where they finish
//     token rows with the shared epilogues (linear_rows.cuh).  While the products run, warps 6-11 ask the epilogue's
//     operands into L2 and run the epilogue's code once with its stores switched off (see the rounds below);
//   * one kernel function serves every epilogue (run-time switch): consecutive launches of a decode step then share their
//     instructions instead of starting cold;
//   * the launch shape (tiles per CTA, K split, ring depth) comes from a small cost model that knows how many clusters of
//     each size the device keeps resident (16 clusters of 8 large CTAs do not fit a B200: such a launch runs in two waves).
// Reference arithmetic replaced: src/ops/matmul.cpp:35-67 -> src/kernels/cpu/matmul.h:10-22 for rows = batch.
#include "linear_rows.cuh"
#include "tcgen05.cuh"

namespace b200 {
namespace {

constexpr int kFeatures = 128;            // features per weight tile (M of the products)
constexpr int kBlockK = 64;               // bf16 columns per stage: one 128-byte swizzle row
constexpr int kWeightBox = kFeatures * kBlockK * 2;   // 16 KB
constexpr int kThreads = 384;             // 12 warps: producer, tensor-core issue, 4 accumulator readers; all 12 finish rows
constexpr int kMaxStages = 8;
constexpr int kControlBytes = 3584;       // barriers, TMEM slot, flags, row scales, row places (position and cache page)
constexpr int kTileStride = kFeatures + 4;
constexpr int kMaxRows = 256;             // two token tiles of 128; above, the prefill kernel (tokens as the M side) takes over
constexpr int kHalfSmem = 113 * 1024;     // two CTAs of this size share an SM

struct DecodeParams {
    LinearParams base;
    int32_t* status;
    int tiles;          // weight tiles per CTA
    int n_pad;          // N of the products: rows rounded up to 16
    int n_alloc;        // tensor-memory columns between two accumulators (power of two >= n_pad)
    int tmem_columns;   // allocation: power of two >= tiles * n_alloc, at least 32
    int stages;
    int body_bytes;     // operand ring (re-used by the epilogue tile), before the control block
    int token_tile;     // activation rows per CTA (grid x walks the token tiles): all rows up to 128, else 128
    int epilogue;       // B200_EPI_*: one kernel serves every epilogue, so that the launches of a step share their code
};

template <int TILES, bool LO, bool QUADS>
__global__ void __launch_bounds__(kThreads, 1) linear_decode_kernel(const __grid_constant__ CUtensorMap map_hi,
                                                                    const __grid_constant__ CUtensorMap map_lo,
                                                                    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ DecodeParams dp) {
    const LinearParams& p = dp.base;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* control = smem + dp.body_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(control);
    uint64_t* empty = full + kMaxStages;
    uint64_t* accumulator_ready = empty + kMaxStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(control + 160);
    volatile int* tile_ready = reinterpret_cast<volatile int*>(control + 192);   // one flag per epilogue warp
    float* row_scale = reinterpret_cast<float*>(control + 256);                  // one per row of the token tile
    int2* row_place = reinterpret_cast<int2*>(control + 1536);                   // q|k|v: position and cache page of every row

    // The warp index goes through a shuffle so that the compiler knows it to be warp-uniform: the role branches below are
    // then uniform control flow, and what the TMA and tensor-core instructions take from uniform registers is computed there.
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int act_bytes = dp.n_pad * kBlockK * 2;
    const int stage_bytes = TILES * kWeightBox + (LO ? 2 : 1) * act_bytes;
    const int tile0 = static_cast<int>(blockIdx.y) * TILES;   // first weight tile of this CTA
    const int row0 = static_cast<int>(blockIdx.x) * dp.token_tile;   // first activation row of this CTA
    const int rows_here = min(dp.token_tile, p.rows - row0);
    // K split: the cluster spans grid z; CTA z of S takes K blocks [k_begin, k_begin + k_blocks), never empty.
    const int split = static_cast<int>(gridDim.z), part = static_cast<int>(blockIdx.z);
    const int all_blocks = (p.in + kBlockK - 1) / kBlockK;
    const int k_begin = all_blocks * part / split, k_blocks = all_blocks * (part + 1) / split - k_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < dp.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accumulator_ready, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, static_cast<uint32_t>(dp.tmem_columns));
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // ---- what the epilogue needs, fixed by the launch (used early by the warm-up pass below) ----
    const int rows_each = (dp.token_tile + split - 1) / split;   // the same for every token tile, so that the slab sizes agree
    const int first = min(rows_here, part * rows_each), last = min(rows_here, first + rows_each);
    const uint32_t slab_bytes = static_cast<uint32_t>(rows_each * kTileStride * 4);
    const uint32_t set_bytes = slab_bytes * static_cast<uint32_t>(split);
    int live_tiles = 0;
    for (int t = 0; t < TILES; ++t) live_tiles += (tile0 + t) * kFeatures < p.out ? 1 : 0;   // the same in every CTA of the cluster
    const bool together = static_cast<uint32_t>(live_tiles) * set_bytes <= static_cast<uint32_t>(dp.body_bytes);
    const uint32_t slabs = smem_u32(smem);

    auto finish_tile = [&](int t, uint32_t set_base, bool whole, int worker) {
        uint32_t partial[8];
#pragma unroll
        for (int z = 0; z < 8; ++z)   // band-relative storage addressed by tile row: shift the base by the band's first row
            partial[z] = set_base + static_cast<uint32_t>(z < split ? z : 0) * slab_bytes - static_cast<uint32_t>(first * kTileStride * 4);
        const float* local = reinterpret_cast<const float*>(smem + (set_base - slabs)) - first * kTileStride;
        const int n0 = (tile0 + t) * kFeatures, workers = kThreads / 32;
        switch (dp.epilogue) {
        case B200_EPI_STORE: finish_rows<B200_EPI_STORE, kFeatures, QUADS ? 1 : 2, true>(p, local, partial, split, row_scale, row0, n0, tile0 + t, first, last, worker, workers, lane, whole); break;
        case B200_EPI_RESIDUAL: finish_rows<B200_EPI_RESIDUAL, kFeatures, QUADS ? 1 : 2, true>(p, local, partial, split, row_scale, row0, n0, tile0 + t, first, last, worker, workers, lane, whole); break;
        case B200_EPI_SWIGLU: finish_rows<B200_EPI_SWIGLU, kFeatures, QUADS ? 1 : 2, true>(p, local, partial, split, row_scale, row0, n0, tile0 + t, first, last, worker, workers, lane, whole); break;
        case B200_EPI_QKV: finish_rows<B200_EPI_QKV, kFeatures, QUADS ? 1 : 2, true>(p, local, partial, split, row_scale, row0, n0, tile0 + t, first, last, worker, workers, lane, whole, row_place); break;
        default: finish_rows<B200_EPI_ARGMAX, kFeatures, QUADS ? 1 : 2, true>(p, local, partial, split, row_scale, row0, n0, tile0 + t, first, last, worker, workers, lane, whole); break;
        }
    };

    if (warp == 0) {
        // TMA producer: the whole warp walks the loop, one elected lane issues.
        if (elect_one()) {
            tma_prefetch_descriptor(&map_w);
            tma_prefetch_descriptor(&map_hi);
            if (LO) tma_prefetch_descriptor(&map_lo);
        }
        // Ring fill, weights first: they do not depend on the preceding kernel.
        const int ahead = k_blocks < dp.stages ? k_blocks : dp.stages;
        for (int i = 0; i < ahead; ++i) {
            uint8_t* stage = smem + i * stage_bytes;
            const int k0 = (k_begin + i) * kBlockK;
            if (elect_one()) {
                mbar_expect_tx(&full[i], static_cast<uint32_t>(stage_bytes));
                for (int t = 0; t < TILES; ++t) tma_load_2d(stage + t * kWeightBox, &map_w, k0, (tile0 + t) * kFeatures, &full[i]);
            }
        }
        grid_dependency_wait();   // the activation shadow comes from the preceding kernel
        grid_launch_dependents();
        for (int i = 0; i < ahead; ++i) {
            uint8_t* stage = smem + i * stage_bytes + TILES * kWeightBox;
            const int k0 = (k_begin + i) * kBlockK;
            if (elect_one()) {
                tma_load_2d(stage, &map_hi, k0, row0, &full[i]);
                if (LO) tma_load_2d(stage + act_bytes, &map_lo, k0, row0, &full[i]);
            }
        }
        {
            // refills: stage index and parity advance without a division (everything here stays warp-uniform)
            int s = ahead == dp.stages ? 0 : ahead;
            uint32_t parity = 0;   // parity of the `empty` phase that frees the stage for its next fill
            for (int i = ahead; i < k_blocks; ++i) {
                const bool freed = mbar_wait(&empty[s], parity);
                if (!__all_sync(0xffffffffu, freed)) {
                    if (lane == 0) atomicExch(dp.status, B200_DEVICE_TIMEOUT);
                    break;
                }
                uint8_t* stage = smem + s * stage_bytes;
                const int k0 = (k_begin + i) * kBlockK;
                if (elect_one()) {
                    mbar_expect_tx(&full[s], static_cast<uint32_t>(stage_bytes));
                    for (int t = 0; t < TILES; ++t) tma_load_2d(stage + t * kWeightBox, &map_w, k0, (tile0 + t) * kFeatures, &full[s]);
                    tma_load_2d(stage + TILES * kWeightBox, &map_hi, k0, row0, &full[s]);
                    if (LO) tma_load_2d(stage + TILES * kWeightBox + act_bytes, &map_lo, k0, row0, &full[s]);
                }
                if (++s == dp.stages) { s = 0; parity ^= 1u; }
            }
        }
    } else {
        grid_dependency_wait();   // sums of squares, residual, cache lengths come from the preceding kernels
        grid_launch_dependents();
        // What the epilogue will read from global memory is asked into L2 now, while the products run: inside a decode
        // step the attention kernels stream the whole cache through L2 between two projections, so the residual rows
        // and the next norm's weights would otherwise come from DRAM one dependent round trip after the other.
        if (dp.epilogue == B200_EPI_RESIDUAL && warp >= 6) {
            const int band = (dp.token_tile + split - 1) / split;
            const int band_first = min(rows_here, part * band), band_rows = min(rows_here, band_first + band) - band_first;
            const int lines_per_row = TILES * (kFeatures * 4 / 128);
            for (int i = static_cast<int>(threadIdx.x) - 192; i < band_rows * lines_per_row; i += kThreads - 192) {
                const int r = i / lines_per_row, line = i - r * lines_per_row;
                const int feature = tile0 * kFeatures + line * 32;
                if (feature < p.out) prefetch_l2(p.residual + static_cast<int64_t>(row0 + band_first + r) * p.out + feature);
            }
            if (p.out_norm_weight && threadIdx.x - 192 < TILES * 4) {
                const int feature = tile0 * kFeatures + (static_cast<int>(threadIdx.x) - 192) * 32;
                if (feature < p.out)
                    prefetch_l2(static_cast<const uint8_t*>(p.out_norm_weight) + static_cast<int64_t>(feature) * (p.out_norm_dtype == B200_BF16 ? 2 : 4));
            }
        }
    }

    if (warp == 1) {
        // Tensor-core issue: the whole warp walks the loop, one elected lane (always the same) issues and commits.
        const uint32_t instruction = mma_instruction_bf16(kFeatures, dp.n_pad);
        bool alive = true;
        int s = 0;
        uint32_t parity = 0;
        const uint32_t ring = smem_u32(smem);
        const uint64_t act_offset = static_cast<uint64_t>((TILES * kWeightBox) >> 4), lo_offset = static_cast<uint64_t>(act_bytes >> 4);
        for (int i = 0; i < k_blocks; ++i) {
            const bool landed = mbar_wait(&full[s], parity);
            if (!__all_sync(0xffffffffu, landed)) {
                if (lane == 0) atomicExch(dp.status, B200_DEVICE_TIMEOUT);
                alive = false;
                break;
            }
            tc_fence_after_sync();
            // Descriptors of a stage differ only in the start-address field (16-byte units, below 2^14 for any shared-memory
            // address), so the tiles, planes and K slices are reached by adding to the stage's first descriptor.
            const uint64_t first = operand_descriptor(ring + static_cast<uint32_t>(s * stage_bytes));
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k) {
                    // advancing the start address by 32 bytes selects the next 16 columns inside the swizzled rows
                    const uint64_t hi = first + act_offset + 2 * k;
#pragma unroll
                    for (int t = 0; t < TILES; ++t) {
                        const uint64_t w = first + static_cast<uint64_t>(t * (kWeightBox >> 4)) + 2 * k;
                        const uint32_t accumulator = tmem_base + static_cast<uint32_t>(t * dp.n_alloc);
                        tc_mma_bf16(accumulator, w, hi, instruction, (i | k) != 0);
                        if (LO) tc_mma_bf16(accumulator, w, hi + lo_offset, instruction, 1);
                    }
                }
                tc_commit(&empty[s]);   // the stage may be refilled once these products have read it
            }
            if (++s == dp.stages) { s = 0; parity ^= 1u; }
        }
        if (alive && elect_one()) tc_commit(accumulator_ready);
    }

    // ---- epilogue ----
    // Warp w may touch TMEM lanes 32 * (w % 4) .. + 31 = features of the weight tile; a thread holds one feature and
    // reads 32 tokens per instruction.  The token rows are divided over the cluster's CTAs (all of them here without a K
    // split).  Every CTA PUSHES its partial accumulators, transposed, into the shared memory of the CTA that owns the
    // token: slab [sender][row of the owner's band][feature] (for a fixed token the lanes of a warp write consecutive
    // features; remote stores do not wait for anything).  After one barrier over the cluster every CTA finds the partial
    // sums of its band in its own shared memory, adds them in sender order (results do not depend on timing) and
    // finishes its rows with all twelve warps, lanes across the features (linear_rows.cuh).  When the slabs of all weight
    // tiles fit the drained operand ring there is one barrier per launch and no CTA is written to after it; otherwise
    // the tiles take turns and a second barrier frees the slabs for the next one.
    const bool finisher = warp >= 2 && warp < 6;   // the four warps that prepare the rows' scales (and cache places)
    const int quarter = warp & 3;
    bool ready = false;
    if (finisher) {
        for (int row = static_cast<int>(threadIdx.x) - 64; row < rows_here; row += 128) {
            float scale = 1.0f;
            if (p.sumsq_in) {
                float total = 0.0f;
                for (int i = 0; i < p.parts_in; ++i) total += __ldg(p.sumsq_in + static_cast<int64_t>(i) * p.rows + row0 + row);
                scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.in)), static_cast<float>(p.eps))));
            }
            row_scale[row] = scale;
            if (dp.epilogue == B200_EPI_QKV) {
                const int2 place = qkv_row_place(p, row0 + row);
                row_place[row] = place;
                if (place.x < p.context) {   // the row's rotation factors, wanted by the epilogue (head_dim / 2 floats each)
                    const int64_t at = static_cast<int64_t>(place.x) * (p.head_dim >> 1);
                    for (int offset = 0; offset < (p.head_dim >> 1); offset += 32) {
                        prefetch_l2(p.cosine + at + offset);
                        prefetch_l2(p.sine + at + offset);
                    }
                }
            }
        }
    }
    // Every warp takes part in draining the accumulators: warp w may read the TMEM lanes 32 * (w % 4) .. + 31, so three
    // warps share each lane quarter and divide the token columns among themselves.
    const int third = warp >> 2;
    auto push_tile = [&](int t, uint32_t set_base) {
        if (!ready) return;
        const uint32_t source = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(t * dp.n_alloc);
        // my slab inside the owner's set, at this thread's feature column
        const uint32_t mine = set_base + static_cast<uint32_t>(part) * slab_bytes + static_cast<uint32_t>(quarter * 32 + lane) * 4;
        if (split == 1) {   // no peers: plain stores into this CTA's tile
            float* column = reinterpret_cast<float*>(smem + (mine - slabs));
#pragma unroll 1
            for (int c = third * 32; c < dp.n_pad; c += 96) {
                uint32_t r[32];
                tmem_load_32(source + static_cast<uint32_t>(c), r);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (c + j < rows_here) column[(c + j) * kTileStride] = __uint_as_float(r[j]);
            }
            return;
        }
#pragma unroll 1
        for (int c = third * 32; c < dp.n_pad; c += 96) {
            int owner = c / rows_each, band_row = c - owner * rows_each;
            uint32_t target = map_peer_shared(mine, static_cast<uint32_t>(owner < split ? owner : 0));
            uint32_t r[32];
            tmem_load_32(source + static_cast<uint32_t>(c), r);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (c + j < rows_here) {
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(target + static_cast<uint32_t>(band_row * kTileStride * 4)), "f"(__uint_as_float(r[j])) : "memory");
                    if (++band_row == rows_each) {
                        band_row = 0;
                        ++owner;
                        if (owner < split) target = map_peer_shared(mine, static_cast<uint32_t>(owner));
                    }
                }
            }
        }
    };
    auto barrier_all = [&]() {
        __syncwarp();
        if (split > 1) cluster_sync_all();
        else __syncthreads();
    };

    bool whole = true;   // read after a round's first barrier: every warp has posted its flag by then
    auto read_flags = [&]() {
        whole = true;
        for (int w = 0; w < kThreads / 32; ++w) whole = whole && tile_ready[w] != 0;
    };
    // Two rounds over the same code.  Round 0, warps 6-11 only, while the products still run: the row epilogue once with
    // every store switched off (accumulators "not valid"), on whatever the shared-memory tile holds.  Inside a decode step
    // the kernels before this one have pushed this code out of the instruction caches and, with the attention kernels
    // streaming the whole cache, out of L2; fetched only when the products were done it stretched the epilogue to two or
    // three times its warm duration.  Round 1 is the epilogue proper.
#pragma unroll 1
    for (int round = (warp >= 6 && live_tiles > 0 && first < last) ? 0 : 1; round < 2; ++round) {
        const bool real = round == 1;
        if (real) {
            ready = mbar_wait_relaxed(accumulator_ready, 0);
            if (!ready && lane == 0) atomicExch(dp.status, B200_DEVICE_TIMEOUT);
            tc_fence_after_sync();
            if (lane == 0) tile_ready[warp] = ready ? 1 : 0;
            if (split > 1) {
                // The slabs lie in the operand ring: a peer may only write into this CTA once the ring is drained, which is
                // when the accumulators are complete.  Every warp has waited for that; the cluster meets before the pushes.
                __syncwarp();
                cluster_sync_all();
            }
        }
        const int tiles_now = real ? live_tiles : 1;
#pragma unroll 1
        for (int t = 0; t < tiles_now; ++t) {
            if (real && (t == 0 || !together)) {
                // all tile sets fit the drained ring: one barrier per launch; otherwise the tiles take turns
                const int from = together ? 0 : t, to = together ? live_tiles : t + 1;
#pragma unroll 1
                for (int u = from; u < to; ++u) push_tile(u, together ? slabs + static_cast<uint32_t>(u) * set_bytes : slabs);
                barrier_all();   // every partial sum of this CTA's band has arrived
                read_flags();
            }
            finish_tile(t, together ? slabs + static_cast<uint32_t>(t) * set_bytes : slabs, real && whole, real ? warp : warp - 6);
            if (real && !together) barrier_all();   // the slabs may be overwritten by the next tile's partial sums
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, static_cast<uint32_t>(dp.tmem_columns));
    }
}

int encode_box(CUtensorMap* map, const void* base, int rows, int columns, int box_rows) {
    encode_tiled_fn encode = tensor_map_encoder();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return B200_NO_DEVICE; }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(columns), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(columns) * 2};
    const cuuint32_t box[2] = {kBlockK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult result = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                   element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(operand) failed with %d", static_cast<int>(result)); return B200_BAD_ARGUMENT; }
    return B200_OK;
}

int round_up_pow2(int value, int least) {
    int result = least;
    while (result < value) result <<= 1;
    return result;
}

}  // namespace

// Clusters of `split` CTAs that can be resident at once, with one CTA per SM (shared memory above half an SM's) or two.
// Asked of the runtime once per (size, residency) and kept; the fallback figures are those of a 148-SM B200.
int cluster_capacity(int split, bool two_per_sm, int sms) {
    static std::mutex mutex;
    static int cached[2][9];
    static const int fallback[2][9] = {{0, 148, 74, 45, 33, 26, 22, 15, 15}, {0, 296, 148, 93, 71, 56, 45, 37, 33}};
    if (split < 1 || split > 8) return 0;
    std::lock_guard<std::mutex> lock(mutex);
    int& slot = cached[two_per_sm ? 1 : 0][split];
    if (slot) return slot;
    auto kernel = linear_decode_kernel<1, true, true>;
    const int smem = two_per_sm ? kHalfSmem : 232448;
    int clusters = 0;
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(1, 16, static_cast<unsigned>(split));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = static_cast<size_t>(smem);
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 1; attribute.val.clusterDim.y = 1; attribute.val.clusterDim.z = static_cast<unsigned>(split);
    config.attrs = &attribute;
    config.numAttrs = 1;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448) != cudaSuccess
        || cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters <= 0) {
        cudaGetLastError();
        clusters = fallback[two_per_sm ? 1 : 0][split] * sms / 148;
    }
    slot = clusters > 0 ? clusters : 1;
    return slot;
}

// Shape of a launch: weight tiles per CTA, K split, ring depth, one or two CTAs per SM.  Every candidate is priced with a
// small model of the kernel (figures measured on B200: a CTA's prologue and epilogue, the shared-memory fill rate of an
// SM, the cost of a tcgen05.mma by its N, resident clusters per cluster size) and the cheapest one is taken.
DecodeShape linear_decode_shape(int rows, int in, int out, bool two_planes, int sms) {
    DecodeShape best{};
    if (rows < 1 || rows > kMaxRows || in <= 0 || out <= 0) return best;
    const int token_tile = rows > 128 ? 128 : rows, token_tiles = (rows + token_tile - 1) / token_tile;
    int n_pad = (token_tile + 15) & ~15;
    if (n_pad < 16) n_pad = 16;
    const int n_alloc = round_up_pow2(n_pad, 32);
    const int feature_tiles = (out + kFeatures - 1) / kFeatures;
    const int k_blocks = (in + kBlockK - 1) / kBlockK;
    const int planes = two_planes ? 2 : 1;
    const int act_bytes = planes * n_pad * kBlockK * 2;
    const int most = 512 / n_alloc < 4 ? 512 / n_alloc : 4;
    const double mma_us = (n_pad <= 64 ? 48.0 : n_pad * 0.5) / 1900.0;   // one product of 128 features x n_pad tokens x 16
    double best_cost = 1e30;
    for (int tiles = 1; tiles <= most; tiles <<= 1) {
        const int groups = (feature_tiles + tiles - 1) / tiles;
        const int stage_bytes = tiles * kWeightBox + act_bytes;
        for (int split = 1; split <= 8; ++split) {
            if (split > 1 && split > k_blocks / 2) break;
            const int per_cta = (k_blocks + split - 1) / split;
            const int rows_each = (token_tile + split - 1) / split;
            const int slab_set = split * rows_each * kTileStride * 4;
            for (int two = 0; two < 2; ++two) {
                const int room = (two ? kHalfSmem : 232448) - 1024 - kControlBytes;
                if (slab_set > room) continue;
                if (two && tiles * n_alloc > 256) continue;   // two CTAs share the 512 columns of tensor memory
                int stages = room / stage_bytes;
                if (stages > kMaxStages) stages = kMaxStages;
                if (stages > per_cta) stages = per_cta;
                if (stages < (per_cta < 2 ? per_cta : 2)) continue;
                const int clusters = groups * token_tiles;
                const int capacity = cluster_capacity(split, two != 0, sms);
                const int waves = (clusters + capacity - 1) / capacity;
                // CTAs that share an SM share its fill rate and its tensor core
                const int sharing = two && clusters * split > sms ? 2 : 1;
                const double in_flight = static_cast<double>(stages) * stage_bytes;
                // fill rate of one CTA: what an SM sustains, unless too few bytes are in flight for the memory latency
                double rate = 140e3 / sharing;                        // bytes per microsecond
                if (in_flight / 1.2 < rate) rate = in_flight / 1.2;   // ~1.2 us from request to arrival under load
                const double load_us = static_cast<double>(per_cta) * stage_bytes / rate;
                const double tensor_us = static_cast<double>(per_cta) * tiles * planes * 4 * mma_us * sharing;
                const double epilogue_us = 1.0 + 0.012 * token_tile * tiles + (split > 1 ? 1.5 + 0.02 * (token_tile - rows_each) * tiles : 0.0);
                double cost = waves * (2.0 + (load_us > tensor_us ? load_us : tensor_us) + epilogue_us);
                // all weights cross HBM once: no shape goes below that
                const double floor_us = static_cast<double>(in) * out * 2 / 6.0e6;
                if (cost < floor_us + 3.0) cost = floor_us + 3.0 + 0.01 * cost;
                if (cost < best_cost) {
                    best_cost = cost;
                    best.tiles = tiles; best.split = split; best.ctas = groups; best.stages = stages; best.stage_bytes = stage_bytes;
                    best.n_pad = n_pad; best.n_alloc = n_alloc; best.token_tile = token_tile; best.token_tiles = token_tiles;
                    const int body = stages * stage_bytes > slab_set ? stages * stage_bytes : slab_set;
                    best.body_bytes = (body + 1023) & ~1023;
                    best.smem_bytes = 1024 + best.body_bytes + kControlBytes;
                    best.tmem_columns = round_up_pow2(tiles * n_alloc, 32);
                }
            }
        }
    }
    return best;
}

int linear_decode_parts(int rows, int in, int out) {
    (void)rows; (void)in;
    return (out + kFeatures - 1) / kFeatures;   // one partial per weight tile: a token row of a tile is finished by one CTA
}

bool linear_decode_takes(int rows) { return rows >= 1 && rows <= kMaxRows; }

namespace {

template <int TILES, bool LO, bool QUADS>
int launch_decode_as(const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const DecodeParams& dp, const DecodeShape& shape,
                     cudaStream_t stream) {
    auto kernel = linear_decode_kernel<TILES, LO, QUADS>;
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    const dim3 grid(static_cast<unsigned>(shape.token_tiles), static_cast<unsigned>(shape.ctas), static_cast<unsigned>(shape.split));
    if (shape.split == 1)
        return cuda_status(launch_dependent(kernel, grid, dim3(kThreads), static_cast<size_t>(shape.smem_bytes), stream, hi, lo, w, dp),
                           "linear_decode_kernel launch");
    return cuda_status(launch_dependent_cluster(kernel, grid, dim3(kThreads), static_cast<size_t>(shape.smem_bytes), stream,
                                                dim3(1, 1, static_cast<unsigned>(shape.split)), hi, lo, w, dp),
                       "linear_decode_kernel cluster launch");
}

template <int TILES, bool LO>
int launch_decode_form(const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const DecodeParams& dp, const DecodeShape& shape,
                       bool quads, cudaStream_t stream) {
    return quads ? launch_decode_as<TILES, LO, true>(hi, lo, w, dp, shape, stream) : launch_decode_as<TILES, LO, false>(hi, lo, w, dp, shape, stream);
}

// Whether the epilogue may address its matrices four features at a time (width and alignment, see rows_take_quads).
bool epilogue_takes_quads(const LinearParams& p, int epilogue) {
    switch (epilogue) {
    case B200_EPI_STORE: return rows_take_quads<B200_EPI_STORE>(p);
    case B200_EPI_RESIDUAL: return rows_take_quads<B200_EPI_RESIDUAL>(p);
    case B200_EPI_SWIGLU: return rows_take_quads<B200_EPI_SWIGLU>(p);
    case B200_EPI_QKV: return rows_take_quads<B200_EPI_QKV>(p);
    default: return rows_take_quads<B200_EPI_ARGMAX>(p);
    }
}

int launch_decode(const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const DecodeParams& dp, const DecodeShape& shape,
                  cudaStream_t stream) {
    const bool two = dp.base.x_lo != nullptr, quads = epilogue_takes_quads(dp.base, dp.epilogue);
    switch (shape.tiles) {
    case 1: return two ? launch_decode_form<1, true>(hi, lo, w, dp, shape, quads, stream) : launch_decode_form<1, false>(hi, lo, w, dp, shape, quads, stream);
    case 2: return two ? launch_decode_form<2, true>(hi, lo, w, dp, shape, quads, stream) : launch_decode_form<2, false>(hi, lo, w, dp, shape, quads, stream);
    case 4: return two ? launch_decode_form<4, true>(hi, lo, w, dp, shape, quads, stream) : launch_decode_form<4, false>(hi, lo, w, dp, shape, quads, stream);
    }
    return B200_UNSUPPORTED;
}

}  // namespace

int launch_linear_decode(const LinearParams& p, int epilogue, cudaStream_t stream) {
    if (p.weight_dtype != B200_BF16 || !p.x_hi || (p.in & 7) || (p.out_hi && (p.out & 1)) || !linear_decode_takes(p.rows)
        || ((reinterpret_cast<uintptr_t>(p.weight) | reinterpret_cast<uintptr_t>(p.x_hi) | reinterpret_cast<uintptr_t>(p.x_lo)) & 15))
        return B200_UNSUPPORTED;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    int32_t* status_word = device_status_word(device);
    if (!status_word) { set_error("the device status word could not be allocated"); return B200_NO_DEVICE; }
    const DecodeShape shape = linear_decode_shape(p.rows, p.in, p.out, p.x_lo != nullptr, sm_count(device));
    if (shape.tiles == 0 || shape.smem_bytes > 232448) return B200_UNSUPPORTED;
    DecodeParams dp{p, status_word, shape.tiles, shape.n_pad, shape.n_alloc, shape.tmem_columns, shape.stages, shape.body_bytes, shape.token_tile, epilogue};
    alignas(64) CUtensorMap hi, lo, w;
    int status = encode_box(&hi, p.x_hi, p.rows, p.in, shape.n_pad);
    if (status == B200_OK) status = encode_box(&lo, p.x_lo ? p.x_lo : p.x_hi, p.rows, p.in, shape.n_pad);
    if (status == B200_OK) status = encode_box(&w, p.weight, p.out, p.in, kFeatures);
    if (status != B200_OK) return status;
    if (epilogue < B200_EPI_STORE || epilogue > B200_EPI_ARGMAX) return B200_UNSUPPORTED;
    return launch_decode(hi, lo, w, dp, shape, stream);
}

}  // namespace b200
