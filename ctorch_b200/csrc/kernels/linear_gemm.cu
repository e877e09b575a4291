// Dense projection for many activation rows (prefill, large decode batches): y = epilogue(scale_rows(x @ W^T)) on the
// 5th-generation tensor cores.  x arrives as an activation shadow (bf16 hi + lo planes, see linear_common.cuh), W is
// bf16 [out, in]; both operands are K-major, the accumulator is f32 in tensor memory.
//
// One CTA computes a 128-token x 128-feature tile:
//   warp 0      TMA producer: per 64-wide K block three 16 KB boxes (x_hi, x_lo, W), 128-byte swizzle, 4-stage
//               mbarrier ring (cp.async.bulk.tensor.2d, no multicast)
//   warp 1      allocates 128 TMEM columns and issues tcgen05.mma.cta_group::1.kind::f16 (M 128, N 128, K 16):
//               D += x_hi.W and D += x_lo.W for the four K slices of a block, then tcgen05.commit releases the
//               stage; a last commit publishes the accumulator
//   warps 2-5   epilogue: tcgen05.ld (32 lanes x 32 columns per instruction) brings each warp's quarter of the
//               accumulator to registers, one token row per thread, and from there to a row-major tile in shared
//               memory; the warps then walk the rows with their lanes across the features, so every global access is
//               coalesced; rows are scaled by the split RMSNorm factor and finished by the shared epilogue (store | residual | SiLU(gate)*up | q|k|v + RoPE + KV append), with
//               the optional output shadow and its per-row sums of squares.
// Few tiles (decode batches of 17..256 rows against a narrow projection) leave most SMs idle and the launch far from
// the HBM rate, so such launches split K over a thread-block cluster of up to 8 CTAs (grid z): every CTA accumulates
// its K range in its own tensor memory, copies the f32 partial tile to its shared memory (the operand ring is free by
// then), and after a cluster barrier each CTA sums a band of rows of the tile over all peers (distributed shared
// memory, fixed order z = 0..S-1, so results do not depend on timing) and runs the epilogue on that band.
// Reference arithmetic replaced: src/ops/matmul.cpp:35-67 -> src/kernels/cpu/matmul.h:10-22 for rows = batch * length.
#include "linear_rows.cuh"
#include "tcgen05.cuh"

namespace b200 {
namespace {

constexpr int kTileM = 128;   // tokens
// features per tile: 128 or 256 (template parameter TN).  The wide tile halves the activation bytes a CTA pulls from L2
// per weight byte, which is what bounds this kernel once the weights stream at HBM rate.
constexpr int kBlockK = 64;   // bf16 columns per stage: one 128-byte swizzle row
constexpr int kBoxBytes = kTileM * kBlockK * 2;  // 16 KB: one activation plane of a K block
template <int TN, int STAGES> struct GemmShape {
    static constexpr int stages = STAGES;
    static constexpr int weight_bytes = TN * kBlockK * 2;
    static constexpr int stage_bytes = 2 * kBoxBytes + weight_bytes;   // x_hi, x_lo, W: 48 KB or 64 KB
    static constexpr int smem = stages * stage_bytes + 1024 + 2048;   // alignment slack; barriers, TMEM slot, 128 row scales, 128 row places
    // Instruction descriptor: f32 accumulator, bf16 x bf16, both K-major, N = TN, M = 128.
    static constexpr uint32_t instruction = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(TN >> 3) << 17)
                                            | (static_cast<uint32_t>(kTileM >> 4) << 24);
};
constexpr int kGemmThreads = 192;

struct GemmParams {
    LinearParams base;
    int32_t* status;
};

template <int EPI, int TN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, STAGES == 2 && TN == 128 ? 2 : 1) linear_gemm_kernel(const __grid_constant__ CUtensorMap map_hi,
                                                                      const __grid_constant__ CUtensorMap map_lo,
                                                                      const __grid_constant__ CUtensorMap map_w, const GemmParams gp) {
    using S = GemmShape<TN, STAGES>;
    constexpr int kStages = S::stages, kStageBytes = S::stage_bytes, kTileN = TN;
    constexpr uint32_t kInstruction = S::instruction;
    const LinearParams& p = gp.base;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* accumulator_ready = empty + kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accumulator_ready + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * kTileM, n0 = blockIdx.y * kTileN;
    // K split: the cluster spans grid z; CTA z of S takes k blocks [k_begin, k_end), never empty (S <= k blocks).
    const int split = static_cast<int>(gridDim.z), part = static_cast<int>(blockIdx.z);
    const int all_blocks = (p.in + kBlockK - 1) / kBlockK;
    const int k_begin = all_blocks * part / split, k_blocks = all_blocks * (part + 1) / split - k_begin;
    const bool has_lo = p.x_lo != nullptr;   // without the lo plane the activations count as bf16 (half the operand bytes and products)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accumulator_ready, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTileN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    grid_dependency_wait();   // the shadow (and residual, cache, sums of squares) come from the preceding kernels
    grid_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_descriptor(&map_hi);
            tma_prefetch_descriptor(&map_lo);
            tma_prefetch_descriptor(&map_w);
            for (int i = 0; i < k_blocks; ++i) {
                const int s = i % kStages;
                const uint32_t phase = (i / kStages) & 1;
                if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(gp.status, B200_DEVICE_TIMEOUT); break; }
                uint8_t* stage = smem + s * kStageBytes;
                const int k0 = (k_begin + i) * kBlockK;
                mbar_expect_tx(&full[s], has_lo ? kStageBytes : kStageBytes - kBoxBytes);
                tma_load_2d(stage, &map_hi, k0, m0, &full[s]);
                if (has_lo) tma_load_2d(stage + kBoxBytes, &map_lo, k0, m0, &full[s]);
                tma_load_2d(stage + 2 * kBoxBytes, &map_w, k0, n0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool alive = true;
            for (int i = 0; i < k_blocks && alive; ++i) {
                const int s = i % kStages;
                const uint32_t phase = (i / kStages) & 1;
                if (!mbar_wait(&full[s], phase)) { atomicExch(gp.status, B200_DEVICE_TIMEOUT); alive = false; break; }
                tc_fence_after_sync();
                const uint32_t stage = smem_u32(smem + s * kStageBytes);
                const uint64_t hi = operand_descriptor(stage), lo = operand_descriptor(stage + kBoxBytes);
                const uint64_t w = operand_descriptor(stage + 2 * kBoxBytes);
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k) {
                    // advancing the start address by 32 bytes selects the next 16 columns inside the swizzled rows
                    tc_mma_bf16(tmem_base, hi + 2 * k, w + 2 * k, kInstruction, (i | k) != 0);
                    if (has_lo) tc_mma_bf16(tmem_base, lo + 2 * k, w + 2 * k, kInstruction, 1);
                }
                tc_commit(&empty[s]);   // the stage may be refilled once these products have read it
            }
            if (alive) tc_commit(accumulator_ready);
        }
    }

    // ---- epilogue, warps 2-5 ----
    // (1) Each warp may touch TMEM lanes 32 * (warp % 4) .. + 31: thread = one token row copies its accumulators to a
    //     row-major f32 tile in shared memory (the drained operand ring; rows padded by 4 floats so that the 16-byte
    //     stores of a quarter warp hit distinct banks).
    // (2) With a K split, a cluster barrier publishes every CTA's partial tile.
    // (3) The rows of the tile are divided over the cluster's CTAs and over the four warps; a warp finishes one row
    //     at a time with its lanes across the feature pairs, so the sums over the peers' tiles (distributed shared
    //     memory, fixed order) and every global access of the epilogue (residual, result, shadows, cache) are
    //     coalesced.  Per-row reductions (sum of squares, argmax candidate) are butterflies.
    constexpr int kTileStride = kTileN + 4;
    float* tile = reinterpret_cast<float*>(smem);
    float* row_scale = reinterpret_cast<float*>(smem + kStages * kStageBytes + 512);   // 128 floats behind the barriers
    int2* row_place = reinterpret_cast<int2*>(smem + kStages * kStageBytes + 1024);    // q|k|v: position and cache page of every row
    volatile int* tile_ready = reinterpret_cast<volatile int*>(smem + kStages * kStageBytes + 256);   // one flag per epilogue warp
    const bool finisher = warp >= 2;
    const int quarter = warp & 3;
    bool ready = false;
    if (finisher) {
        const int tile_row = quarter * 32 + lane;
        const int row = m0 + tile_row;
        float scale = 1.0f;
        if (p.sumsq_in && row < p.rows) {
            float total = 0.0f;
            for (int i = 0; i < p.parts_in; ++i) total += __ldg(p.sumsq_in + static_cast<int64_t>(i) * p.rows + row);
            scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.in)), static_cast<float>(p.eps))));
        }
        row_scale[tile_row] = scale;
        if constexpr (EPI == B200_EPI_QKV) row_place[tile_row] = qkv_row_place(p, row);
        ready = mbar_wait(accumulator_ready, 0);
        if (!ready && lane == 0) atomicExch(gp.status, B200_DEVICE_TIMEOUT);
        tc_fence_after_sync();
        if (ready) {
#pragma unroll 1
            for (int c = 0; c < kTileN / 32; ++c) {
                uint32_t r[32];
                tmem_load_32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, r);
                float4* out4 = reinterpret_cast<float4*>(tile + tile_row * kTileStride + c * 32);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    out4[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                          __uint_as_float(r[4 * j + 3]));
            }
        }
        if (lane == 0) tile_ready[quarter] = ready ? 1 : 0;
    }
    __syncwarp();
    if (split > 1) cluster_sync_all();   // every CTA's partial tile is complete and visible to its peers
    else __syncthreads();                // the whole tile is in shared memory
    {
        // All six warps finish rows (the producer and the issuing warp are idle by now).  Only rows that exist are divided
        // over the cluster's CTAs: a decode batch of 32 rows keeps every CTA of the cluster busy.
        ready = tile_ready[0] && tile_ready[1] && tile_ready[2] && tile_ready[3];
        const int rows_here = min(kTileM, p.rows - m0);
        const int rows_each = (rows_here + split - 1) / split;
        const int first = part * rows_each, last = min(rows_here, first + rows_each);
        uint32_t peer_tile[8];
        peer_tile[0] = smem_u32(tile);
        if (split > 1) {
#pragma unroll
            for (int z = 0; z < 8; ++z) peer_tile[z] = z < split ? map_peer_shared(smem_u32(tile), static_cast<uint32_t>(z)) : 0u;
        }
        finish_rows<EPI, kTileN>(p, tile, peer_tile, split, row_scale, m0, n0, static_cast<int>(blockIdx.y), first, last, warp, kGemmThreads / 32, lane, ready,
                                 EPI == B200_EPI_QKV ? row_place : nullptr);
    }
    if (split > 1) {
        __syncwarp();
        cluster_sync_all();   // no CTA leaves while a peer may still read its shared memory
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTileN);
    }
}

// ---- persistent variant: more tiles than SMs, no K split -----------------------------------------------------------
// One CTA per SM walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (token tile fastest, so neighbouring CTAs share
// a weight tile).  The accumulator is double-buffered in tensor memory (2 x 128 columns) and the epilogue has its own
// shared-memory tile next to a 3-stage operand ring, so warps 2-5 finish tile j while the producer and the issuing
// thread are already streaming and multiplying tile j + 1: the tensor pipe does not idle during epilogues and the ring
// never drains between tiles.
constexpr int kPersistStages = 3;
constexpr int kPersistStageBytes = 3 * kBoxBytes;                      // x_hi, x_lo, W boxes of one K block: 48 KB
constexpr int kPersistTileBytes = kTileM * (128 + 4) * 4;              // row-major f32 tile of the epilogue, padded rows
constexpr int kPersistSmem = kPersistStages * kPersistStageBytes + kPersistTileBytes + 1024 + 2048;
constexpr uint32_t kPersistInstruction = GemmShape<128, 3>::instruction;

template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1) linear_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_hi,
                                                                                 const __grid_constant__ CUtensorMap map_lo,
                                                                                 const __grid_constant__ CUtensorMap map_w,
                                                                                 const GemmParams gp, const int row_tiles, const int tiles) {
    constexpr int kTileN = 128, kTileStride = kTileN + 4;
    const LinearParams& p = gp.base;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    float* tile = reinterpret_cast<float*>(smem + kPersistStages * kPersistStageBytes);
    uint8_t* control = smem + kPersistStages * kPersistStageBytes + kPersistTileBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(control);
    uint64_t* empty = full + kPersistStages;
    uint64_t* acc_full = empty + kPersistStages;    // [2] the products of a tile are complete (tcgen05.commit)
    uint64_t* acc_empty = acc_full + 2;             // [2] the epilogue has read the buffer (one arrival per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* alive_flag = reinterpret_cast<volatile int*>(control + 256);
    float* row_scale = reinterpret_cast<float*>(control + 512);
    int2* row_place = reinterpret_cast<int2*>(control + 1024);   // q|k|v: position and cache page of every row of the tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (p.in + kBlockK - 1) / kBlockK;
    const bool has_lo = p.x_lo != nullptr;
    const int my_tiles = (tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPersistStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        *alive_flag = 1;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * kTileN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    grid_dependency_wait();   // the shadow (and residual, cache, sums of squares) come from the preceding kernels
    grid_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_descriptor(&map_hi);
            tma_prefetch_descriptor(&map_lo);
            tma_prefetch_descriptor(&map_w);
            int it = 0;   // K blocks issued so far, over all tiles: the ring does not restart between tiles
            bool alive = true;
            for (int j = 0; j < my_tiles && alive; ++j) {
                const int t = blockIdx.x + j * gridDim.x;
                const int m0 = (t % row_tiles) * kTileM, n0 = (t / row_tiles) * kTileN;
                for (int i = 0; i < k_blocks; ++i, ++it) {
                    const int s = it % kPersistStages;
                    const uint32_t phase = (it / kPersistStages) & 1;
                    if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(gp.status, B200_DEVICE_TIMEOUT); alive = false; break; }
                    uint8_t* stage = smem + s * kPersistStageBytes;
                    mbar_expect_tx(&full[s], has_lo ? kPersistStageBytes : kPersistStageBytes - kBoxBytes);
                    tma_load_2d(stage, &map_hi, i * kBlockK, m0, &full[s]);
                    if (has_lo) tma_load_2d(stage + kBoxBytes, &map_lo, i * kBlockK, m0, &full[s]);
                    tma_load_2d(stage + 2 * kBoxBytes, &map_w, i * kBlockK, n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int j = 0; j < my_tiles && alive; ++j) {
                const int buffer = j & 1;
                // the epilogue of the tile that used this buffer two tiles ago must have read it (passes at once for j < 2)
                if (!mbar_wait(&acc_empty[buffer], ((j >> 1) & 1) ^ 1)) { atomicExch(gp.status, B200_DEVICE_TIMEOUT); break; }
                tc_fence_after_sync();
                const uint32_t accumulator = tmem_base + static_cast<uint32_t>(buffer * kTileN);
                for (int i = 0; i < k_blocks; ++i, ++it) {
                    const int s = it % kPersistStages;
                    const uint32_t phase = (it / kPersistStages) & 1;
                    if (!mbar_wait(&full[s], phase)) { atomicExch(gp.status, B200_DEVICE_TIMEOUT); alive = false; break; }
                    tc_fence_after_sync();
                    const uint32_t stage = smem_u32(smem + s * kPersistStageBytes);
                    const uint64_t hi = operand_descriptor(stage), lo = operand_descriptor(stage + kBoxBytes);
                    const uint64_t w = operand_descriptor(stage + 2 * kBoxBytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        tc_mma_bf16(accumulator, hi + 2 * k, w + 2 * k, kPersistInstruction, (i | k) != 0);
                        if (has_lo) tc_mma_bf16(accumulator, lo + 2 * k, w + 2 * k, kPersistInstruction, 1);
                    }
                    tc_commit(&empty[s]);
                }
                if (alive) tc_commit(&acc_full[buffer]);
            }
        }
    } else {
        // ---- epilogue warps 2-5: TMEM lanes 32 * (warp % 4) .. + 31; named barrier 2 joins the four warps ----
        const int quarter = warp & 3;
        const int tile_row = quarter * 32 + lane;
        const uint32_t own_tile[8] = {smem_u32(tile), 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        for (int j = 0; j < my_tiles; ++j) {
            const int t = blockIdx.x + j * gridDim.x;
            const int m0 = (t % row_tiles) * kTileM, n0 = (t / row_tiles) * kTileN;
            const int buffer = j & 1;
            const int row = m0 + tile_row;
            float scale = 1.0f;
            if (p.sumsq_in && row < p.rows) {
                float total = 0.0f;
                for (int i = 0; i < p.parts_in; ++i) total += __ldg(p.sumsq_in + static_cast<int64_t>(i) * p.rows + row);
                scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.in)), static_cast<float>(p.eps))));
            }
            row_scale[tile_row] = scale;   // the previous tile's rows were finished before the barrier that ended it
            if constexpr (EPI == B200_EPI_QKV) row_place[tile_row] = qkv_row_place(p, row);
            const bool ready = mbar_wait(&acc_full[buffer], (j >> 1) & 1);
            if (!ready && lane == 0) { atomicExch(gp.status, B200_DEVICE_TIMEOUT); *alive_flag = 0; }
            tc_fence_after_sync();
            if (ready) {
#pragma unroll 1
                for (int c = 0; c < kTileN / 32; ++c) {
                    uint32_t r[32];
                    tmem_load_32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buffer * kTileN + c * 32), r);
                    float4* out4 = reinterpret_cast<float4*>(tile + tile_row * kTileStride + c * 32);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        out4[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                              __uint_as_float(r[4 * q + 3]));
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buffer]);   // the issuing thread may reuse this accumulator
            asm volatile("bar.sync 2, 128;" ::: "memory");    // the tile (and the row scales) are in shared memory
            if (*alive_flag == 0) break;                       // same decision in all four warps
            const int rows_here = min(kTileM, p.rows - m0);
            finish_rows<EPI, kTileN>(p, tile, own_tile, 1, row_scale, m0, n0, t / row_tiles, 0, rows_here, quarter, 4, lane, true,
                                     EPI == B200_EPI_QKV ? row_place : nullptr);
            asm volatile("bar.sync 2, 128;" ::: "memory");    // the next tile may overwrite the shared-memory tile
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * kTileN);
    }
}

int encode_operand(CUtensorMap* map, const void* base, int rows, int columns, int box_rows) {
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

// Tile width of a launch: 128 features; 256 only for very wide matrices (vocabulary projections), where the tiles still
// fill the SMs several times over and the wide tile halves the activation bytes pulled per weight byte.
// Launches the persistent kernel serves: prefill-sized passes (8 or more token tiles, more tiles than SMs) whose K is short
// enough that the epilogues are a large share of a tile's time (measured: K 768 +28 %, K 2048 +5 %, K 8192 -11 % against the
// one-tile-per-CTA kernel with the wide tile).
bool takes_persistent(int rows, int in, int out, int sms) {
    const int row_tiles = (rows + kTileM - 1) / kTileM;
    return row_tiles >= 8 && in <= 2048 && row_tiles * ((out + 127) / 128) > sms;
}

int choose_tile_features(int rows, int in, int out) {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) sms = sm_count(device);
    if (takes_persistent(rows, in, out, sms)) return 128;
    const int row_tiles = (rows + kTileM - 1) / kTileM;
    return row_tiles * ((out + 255) / 256) >= 2 * sms ? 256 : 128;
}

// Ring depth for the 128-wide tile: two stages (96 KB) let two CTAs share an SM, so one tile's epilogue and pipeline ramp
// overlap the other's products; up to 64 rows the activation boxes are mostly zero fill and a CTA alone with a deep ring
// streams weights faster.
int choose_stages(int rows) { return rows > 64 ? 2 : 4; }

// K split of a launch: cluster CTAs (grid z) while the grid stays within one wave of the SMs, at most 4 (larger clusters
// of CTAs this big place badly), and at least two K blocks per CTA.
int choose_split(int rows, int in, int out) {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) sms = sm_count(device);
    const int tn = choose_tile_features(rows, in, out);
    const int tiles = ((rows + kTileM - 1) / kTileM) * ((out + tn - 1) / tn);
    const int k_blocks = (in + kBlockK - 1) / kBlockK;
    int split = sms / (tiles > 0 ? tiles : 1);
    if (split > 4) split = 4;
    if (split > k_blocks / 2) split = k_blocks / 2;
    return split < 1 ? 1 : split;
}

template <int EPI, int TN, int STAGES>
int launch_gemm(const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const GemmParams& gp, cudaStream_t stream) {
    using S = GemmShape<TN, STAGES>;
    auto kernel = linear_gemm_kernel<EPI, TN, STAGES>;
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::smem));
    const int split = choose_split(gp.base.rows, gp.base.in, gp.base.out);
    const dim3 grid((gp.base.rows + kTileM - 1) / kTileM, (gp.base.out + TN - 1) / TN, split);
    if (split == 1)
        return cuda_status(launch_dependent(kernel, grid, dim3(kGemmThreads), S::smem, stream, hi, lo, w, gp), "linear_gemm_kernel launch");
    return cuda_status(launch_dependent_cluster(kernel, grid, dim3(kGemmThreads), S::smem, stream, dim3(1, 1, split), hi, lo, w, gp),
                       "linear_gemm_kernel cluster launch");
}

template <int TN, int STAGES>
int launch_epilogue(int epilogue, const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const GemmParams& gp, cudaStream_t stream) {
    switch (epilogue) {
    case B200_EPI_STORE: return launch_gemm<B200_EPI_STORE, TN, STAGES>(hi, lo, w, gp, stream);
    case B200_EPI_RESIDUAL: return launch_gemm<B200_EPI_RESIDUAL, TN, STAGES>(hi, lo, w, gp, stream);
    case B200_EPI_SWIGLU: return launch_gemm<B200_EPI_SWIGLU, TN, STAGES>(hi, lo, w, gp, stream);
    case B200_EPI_QKV: return launch_gemm<B200_EPI_QKV, TN, STAGES>(hi, lo, w, gp, stream);
    case B200_EPI_ARGMAX: return launch_gemm<B200_EPI_ARGMAX, TN, STAGES>(hi, lo, w, gp, stream);
    }
    return B200_UNSUPPORTED;
}

}  // namespace

int linear_gemm_parts(int rows, int in, int out) {
    if (linear_decode_takes(rows)) return linear_decode_parts(rows, in, out);
    const int tn = choose_tile_features(rows, in, out);
    return (out + tn - 1) / tn;   // one partial per feature tile: a row of a tile is finished by one CTA of the cluster
}

template <int EPI>
int launch_persistent_epilogue(const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const GemmParams& gp, int row_tiles, int tiles,
                               int sms, cudaStream_t stream) {
    auto kernel = linear_gemm_persistent_kernel<EPI>;
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPersistSmem));
    return cuda_status(launch_dependent(kernel, dim3(static_cast<unsigned>(tiles < sms ? tiles : sms)), dim3(kGemmThreads), kPersistSmem, stream, hi, lo,
                                        w, gp, row_tiles, tiles), "linear_gemm_persistent_kernel launch");
}

int launch_persistent(int epilogue, const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const GemmParams& gp, int row_tiles,
                      int tiles, int sms, cudaStream_t stream) {
    switch (epilogue) {
    case B200_EPI_STORE: return launch_persistent_epilogue<B200_EPI_STORE>(hi, lo, w, gp, row_tiles, tiles, sms, stream);
    case B200_EPI_RESIDUAL: return launch_persistent_epilogue<B200_EPI_RESIDUAL>(hi, lo, w, gp, row_tiles, tiles, sms, stream);
    case B200_EPI_SWIGLU: return launch_persistent_epilogue<B200_EPI_SWIGLU>(hi, lo, w, gp, row_tiles, tiles, sms, stream);
    case B200_EPI_QKV: return launch_persistent_epilogue<B200_EPI_QKV>(hi, lo, w, gp, row_tiles, tiles, sms, stream);
    case B200_EPI_ARGMAX: return launch_persistent_epilogue<B200_EPI_ARGMAX>(hi, lo, w, gp, row_tiles, tiles, sms, stream);
    }
    return B200_UNSUPPORTED;
}

int launch_linear_gemm(const LinearParams& p, int epilogue, cudaStream_t stream) {
    if (linear_decode_takes(p.rows)) return launch_linear_decode(p, epilogue, stream);   // decode batches: weights streamed once
    if (p.weight_dtype != B200_BF16 || !p.x_hi || (p.in & 7) || (p.out_hi && (p.out & 1))
        || ((reinterpret_cast<uintptr_t>(p.weight) | reinterpret_cast<uintptr_t>(p.x_hi) | reinterpret_cast<uintptr_t>(p.x_lo)) & 15))
        return B200_UNSUPPORTED;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    GemmParams gp{p, device_status_word(device)};
    if (!gp.status) { set_error("the device status word could not be allocated"); return B200_NO_DEVICE; }
    alignas(64) CUtensorMap hi, lo, w;
    const int sms = sm_count(device);
    const int row_tiles = (p.rows + kTileM - 1) / kTileM, tiles128 = row_tiles * ((p.out + 127) / 128);
    const bool persistent = takes_persistent(p.rows, p.in, p.out, sms);
    const int tn = persistent ? 128 : choose_tile_features(p.rows, p.in, p.out);
    int status = encode_operand(&hi, p.x_hi, p.rows, p.in, kTileM);
    if (status == B200_OK) status = encode_operand(&lo, p.x_lo ? p.x_lo : p.x_hi, p.rows, p.in, kTileM);
    if (status == B200_OK) status = encode_operand(&w, p.weight, p.out, p.in, tn);
    if (status != B200_OK) return status;
    if (persistent) return launch_persistent(epilogue, hi, lo, w, gp, row_tiles, tiles128, sms, stream);
    const int stages = choose_stages(p.rows);
    if (tn == 256) return launch_epilogue<256, 3>(epilogue, hi, lo, w, gp, stream);
    return stages == 2 ? launch_epilogue<128, 2>(epilogue, hi, lo, w, gp, stream) : launch_epilogue<128, 4>(epilogue, hi, lo, w, gp, stream);
}

}  // namespace b200
