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
//               accumulator to registers, one token row per thread; rows are scaled by the split RMSNorm factor and
//               finished by the shared epilogue (store | residual | SiLU(gate)*up | q|k|v + RoPE + KV append), with
//               the optional output shadow and its per-row sums of squares.
// Few tiles (decode batches of 17..256 rows against a narrow projection) leave most SMs idle and the launch far from
// the HBM rate, so such launches split K over a thread-block cluster of up to 8 CTAs (grid z): every CTA accumulates
// its K range in its own tensor memory, dumps the f32 partial tile to its shared memory (the operand ring is free by
// then), and after a cluster barrier each CTA sums one column slice of the tile over all peers (distributed shared
// memory, fixed order z = 0..S-1, so results do not depend on timing) and runs the epilogue on that slice.
// Reference arithmetic replaced: src/ops/matmul.cpp:35-67 -> src/kernels/cpu/matmul.h:10-22 for rows = batch * length.
#include "linear_common.cuh"

namespace b200 {
namespace {

constexpr int kTileM = 128;   // tokens
constexpr int kTileN = 128;   // features
constexpr int kBlockK = 64;   // bf16 columns per stage: one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kBoxBytes = kTileM * kBlockK * 2;  // 16 KB, same for the three operands
constexpr int kStageBytes = 3 * kBoxBytes;
constexpr int kGemmThreads = 192;
constexpr int kGemmSmem = kStages * kStageBytes + 1024 + 256;

struct GemmParams {
    LinearParams base;
    int32_t* status;
};

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile [rows][64 bf16] written by TMA with 128-byte swizzle:
// 8-row groups of 1024 bytes follow each other (stride byte offset 1024), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t smem_address) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_address & 0x3ffff) >> 4);   // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;                          // descriptor version of this architecture
    d |= static_cast<uint64_t>(2) << 61;                          // 128-byte swizzle
    return d;
}
// Instruction descriptor: f32 accumulator, bf16 x bf16, both K-major, N = 128, M = 128.
constexpr uint32_t kInstruction = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kTileN >> 3) << 17)
                                  | (static_cast<uint32_t>(kTileM >> 4) << 24);

// One finished pair of adjacent features of one token row: shared epilogue, then the optional output shadow (hi + lo of
// the value times the next norm weight) and the running sum of squares of the new residual stream.
template <int EPI>
__device__ __forceinline__ void finish_pair(const LinearParams& p, int row, int feature0, float a, float b, float& squares) {
    linear_epilogue<EPI>(p, row, feature0, a, b);
    if constexpr (EPI == B200_EPI_RESIDUAL) {
        const bool second = feature0 + 1 < p.out;
        squares += a * a + (second ? b * b : 0.0f);
        if (p.out_hi) {
            float wa = 1.0f, wb = 1.0f;
            if (p.out_norm_weight) {
                if (p.out_norm_dtype == B200_BF16) {
                    const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(p.out_norm_weight) + feature0;
                    wa = __bfloat162float(w[0]);
                    wb = second ? __bfloat162float(w[1]) : 0.0f;
                } else {
                    const float* w = static_cast<const float*>(p.out_norm_weight) + feature0;
                    wa = w[0];
                    wb = second ? w[1] : 0.0f;
                }
            }
            const float va = __fmul_rn(a, wa), vb = __fmul_rn(b, wb);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(va, vb);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(va - __low2float(hi), vb - __high2float(hi));
            const int64_t at = static_cast<int64_t>(row) * p.out + feature0;
            *reinterpret_cast<__nv_bfloat162*>(p.out_hi + at) = hi;
            *reinterpret_cast<__nv_bfloat162*>(p.out_lo + at) = lo;
        }
    }
    if constexpr (EPI == B200_EPI_SWIGLU) {
        if (p.out_hi) {
            const __nv_bfloat16 hi = __float2bfloat16_rn(a);
            const int64_t at = static_cast<int64_t>(row) * (p.out >> 1) + (feature0 >> 1);
            p.out_hi[at] = hi;
            p.out_lo[at] = __float2bfloat16_rn(a - __bfloat162float(hi));
        }
    }
}

template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1) linear_gemm_kernel(const __grid_constant__ CUtensorMap map_hi,
                                                                      const __grid_constant__ CUtensorMap map_lo,
                                                                      const __grid_constant__ CUtensorMap map_w, const GemmParams gp) {
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
                mbar_expect_tx(&full[s], kStageBytes);
                tma_load_2d(stage, &map_hi, k0, m0, &full[s]);
                tma_load_2d(stage + kBoxBytes, &map_lo, k0, m0, &full[s]);
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
                    tc_mma_bf16(tmem_base, lo + 2 * k, w + 2 * k, kInstruction, 1);
                }
                tc_commit(&empty[s]);   // the stage may be refilled once these products have read it
            }
            if (alive) tc_commit(accumulator_ready);
        }
    }

    // ---- epilogue warps 2-5: warp w may touch TMEM lanes 32 * (w % 4) .. + 31; thread = one token row ----
    const bool finisher = warp >= 2;
    const int quarter = warp & 3;
    const int tile_row = quarter * 32 + lane;
    const int row = m0 + tile_row;
    float scale = 1.0f, squares = 0.0f;
    Candidate best{-INFINITY, INT32_MAX};   // B200_EPI_ARGMAX: this row's preferred feature among the columns seen so far
    bool ready = false;
    if (finisher) {
        if (p.sumsq_in && row < p.rows) {
            float total = 0.0f;
            for (int i = 0; i < p.parts_in; ++i) total += __ldg(p.sumsq_in + static_cast<int64_t>(i) * p.rows + row);
            scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.in)), static_cast<float>(p.eps))));
        }
        ready = mbar_wait(accumulator_ready, 0);
        if (!ready && lane == 0) atomicExch(gp.status, B200_DEVICE_TIMEOUT);
        tc_fence_after_sync();
    }
    if (split == 1) {
        if (finisher && ready) {
#pragma unroll 1
            for (int c = 0; c < kTileN / 32; ++c) {
                uint32_t r[32];
                tmem_load_32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, r);
                if (row >= p.rows) continue;
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int feature0 = n0 + c * 32 + j;
                    if (feature0 >= p.out) continue;
                    const float a = __uint_as_float(r[j]) * scale, b = __uint_as_float(r[j + 1]) * scale;
                    if constexpr (EPI == B200_EPI_ARGMAX) {
                        const Candidate pair = pair_candidate(feature0, a, b, p.out);
                        if (preferred(pair, best)) best = pair;
                    } else {
                        finish_pair<EPI>(p, row, feature0, a, b, squares);
                    }
                }
            }
            if constexpr (EPI == B200_EPI_RESIDUAL) {
                if (p.sumsq_out && row < p.rows) p.sumsq_out[static_cast<int64_t>(blockIdx.y) * p.rows + row] = squares;
            }
            if constexpr (EPI == B200_EPI_ARGMAX) {
                if (row < p.rows) {
                    p.best_value[static_cast<int64_t>(blockIdx.y) * p.rows + row] = best.value;
                    p.best_index[static_cast<int64_t>(blockIdx.y) * p.rows + row] = best.index;
                }
            }
        }
    } else {
        // Partial tile, transposed [feature column][token row] f32 (64 KB over the first stages of the drained ring):
        // a warp's lanes are consecutive rows, so its stores and the peers' loads are conflict-free and coalesced.
        float* partial = reinterpret_cast<float*>(smem);
        if (finisher && ready) {
#pragma unroll 1
            for (int c = 0; c < kTileN / 32; ++c) {
                uint32_t r[32];
                tmem_load_32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, r);
#pragma unroll
                for (int j = 0; j < 32; ++j) partial[(c * 32 + j) * kTileM + tile_row] = __uint_as_float(r[j]);
            }
        }
        __syncwarp();
        cluster_sync_all();   // every CTA's partial tile is complete and visible to its peers
        if (finisher && ready && row < p.rows) {
            const int width = ((kTileN + split - 1) / split + 1) & ~1;   // even: the epilogues work on feature pairs
            const int c_begin = part * width, c_end = min(kTileN, c_begin + width);
            const uint32_t mine = smem_u32(partial) + static_cast<uint32_t>(tile_row) * 4;
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 2) {
                const int feature0 = n0 + c;
                if (feature0 >= p.out) break;
                float a = 0.0f, b = 0.0f;
                for (int z = 0; z < split; ++z) {
                    a += load_peer_shared(mine + static_cast<uint32_t>(c * kTileM) * 4, static_cast<uint32_t>(z));
                    b += load_peer_shared(mine + static_cast<uint32_t>((c + 1) * kTileM) * 4, static_cast<uint32_t>(z));
                }
                if constexpr (EPI == B200_EPI_ARGMAX) {
                    const Candidate pair = pair_candidate(feature0, a * scale, b * scale, p.out);
                    if (preferred(pair, best)) best = pair;
                } else {
                    finish_pair<EPI>(p, row, feature0, a * scale, b * scale, squares);
                }
            }
            if constexpr (EPI == B200_EPI_RESIDUAL) {
                if (p.sumsq_out) p.sumsq_out[(static_cast<int64_t>(blockIdx.y) * split + part) * p.rows + row] = squares;
            }
            if constexpr (EPI == B200_EPI_ARGMAX) {
                p.best_value[(static_cast<int64_t>(blockIdx.y) * split + part) * p.rows + row] = best.value;
                p.best_index[(static_cast<int64_t>(blockIdx.y) * split + part) * p.rows + row] = best.index;
            }
        }
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

int encode_operand(CUtensorMap* map, const void* base, int rows, int columns) {
    encode_tiled_fn encode = tensor_map_encoder();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return B200_NO_DEVICE; }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(columns), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(columns) * 2};
    const cuuint32_t box[2] = {kBlockK, kTileM};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult result = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                   element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(operand) failed with %d", static_cast<int>(result)); return B200_BAD_ARGUMENT; }
    return B200_OK;
}

// K split of a launch: as many cluster CTAs as keep the grid within one wave of the SMs, at most 8 (the portable
// cluster size), and at least two K blocks per CTA.
int choose_split(int rows, int in, int out) {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) sms = sm_count(device);
    const int tiles = ((rows + kTileM - 1) / kTileM) * ((out + kTileN - 1) / kTileN);
    const int k_blocks = (in + kBlockK - 1) / kBlockK;
    int split = sms / (tiles > 0 ? tiles : 1);
    if (split > 8) split = 8;
    if (split > k_blocks / 2) split = k_blocks / 2;
    return split < 1 ? 1 : split;
}

template <int EPI> int launch_gemm(const CUtensorMap& hi, const CUtensorMap& lo, const CUtensorMap& w, const GemmParams& gp, cudaStream_t stream) {
    auto kernel = linear_gemm_kernel<EPI>;
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem));
    const int split = choose_split(gp.base.rows, gp.base.in, gp.base.out);
    const dim3 grid((gp.base.rows + kTileM - 1) / kTileM, (gp.base.out + kTileN - 1) / kTileN, split);
    if (split == 1)
        return cuda_status(launch_dependent(kernel, grid, dim3(kGemmThreads), kGemmSmem, stream, hi, lo, w, gp), "linear_gemm_kernel launch");
    return cuda_status(launch_dependent_cluster(kernel, grid, dim3(kGemmThreads), kGemmSmem, stream, dim3(1, 1, split), hi, lo, w, gp),
                       "linear_gemm_kernel cluster launch");
}

}  // namespace

int linear_gemm_parts(int rows, int in, int out) { return ((out + kTileN - 1) / kTileN) * choose_split(rows, in, out); }

int launch_linear_gemm(const LinearParams& p, int epilogue, cudaStream_t stream) {
    if (p.weight_dtype != B200_BF16 || !p.x_hi || !p.x_lo || (p.in & 7) || (p.out_hi && (p.out & 1))
        || ((reinterpret_cast<uintptr_t>(p.weight) | reinterpret_cast<uintptr_t>(p.x_hi) | reinterpret_cast<uintptr_t>(p.x_lo)) & 15))
        return B200_UNSUPPORTED;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    GemmParams gp{p, device_status_word(device)};
    alignas(64) CUtensorMap hi, lo, w;
    int status = encode_operand(&hi, p.x_hi, p.rows, p.in);
    if (status == B200_OK) status = encode_operand(&lo, p.x_lo, p.rows, p.in);
    if (status == B200_OK) status = encode_operand(&w, p.weight, p.out, p.in);
    if (status != B200_OK) return status;
    switch (epilogue) {
    case B200_EPI_STORE: return launch_gemm<B200_EPI_STORE>(hi, lo, w, gp, stream);
    case B200_EPI_RESIDUAL: return launch_gemm<B200_EPI_RESIDUAL>(hi, lo, w, gp, stream);
    case B200_EPI_SWIGLU: return launch_gemm<B200_EPI_SWIGLU>(hi, lo, w, gp, stream);
    case B200_EPI_QKV: return launch_gemm<B200_EPI_QKV>(hi, lo, w, gp, stream);
    case B200_EPI_ARGMAX: return launch_gemm<B200_EPI_ARGMAX>(hi, lo, w, gp, stream);
    }
    return B200_UNSUPPORTED;
}

}  // namespace b200
