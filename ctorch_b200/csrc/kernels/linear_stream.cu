// Streaming skinny linear for bf16 weights and up to 16 activation rows per tile (the decode batch):
// y = epilogue(rmsnorm?(x) @ W^T).  The work is weight streaming, so the kernel is built around keeping many
// kilobytes of weights in flight per SM:
//   * persistent CTAs (one per SM) walk feature tiles of TF rows of W; a producer warp streams every tile through
//     a ring of shared-memory slots with bulk TMA copies (cp.async.bulk, one per weight row, mbarrier completion,
//     no multicast, no descriptor to fetch) and runs ahead across tile boundaries; the first slots are requested
//     before the activations are touched, so DRAM latency overlaps the prologue; rows land with a padded stride
//     so that ldmatrix reads them without bank conflicts;
//   * the activation rows are staged once per CTA: RMSNorm in f64 (src/kernels/cpu/normalization.cpp:39-51 of the
//     reference), then split into bf16 hi + bf16 lo so that the tensor cores see ~16 mantissa bits of the f32 value;
//   * eight consumer warps split K: warp w takes the 16-column k-steps w, w+8, ... of every stage, multiplies the
//     [16 x 16] activation fragments (hi and lo) with the [16 x TF] weight fragments using mma.sync m16n8k16 bf16
//     with f32 accumulation (fragments via ldmatrix from the swizzled stage), and the per-warp partial sums are
//     added through shared memory before the shared epilogue (linear_common.cuh) runs.
// Rows beyond 16 are covered by blockIdx.y (weights then come from L2).  Shapes it does not take (f32 weights,
// in > 2048 or in % 8 != 0) stay on the CUDA-core kernel.
#include "linear_common.cuh"

#include <mutex>
#include <type_traits>


namespace b200 {
namespace {

constexpr int kConsumers = 8;
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr int kRows = 16;
constexpr int kMaxIn = 2048;

struct StreamParams {
    LinearParams base;
    int tile_features;   // TF: 8, 16, 32 or 64
    int slots;           // ring depth, one whole tile [TF][in_padded + 8] per slot
    int tiles;           // ceil(out / TF)
    int in_padded;       // in rounded up to 64
    int32_t* status;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(address));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory"); }

// 1-D bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Shared memory map (offsets from a 128-byte aligned base):
//   [0, slots * slot_bytes)         weight tiles, [TF rows][in_padded + 8] bf16 each (row stride = 16 mod 128 bytes)
//   then x_hi, x_lo                 [16][in_padded + 8] bf16 each
//   then partial sums               [8 warps][16 rows][TF] f32
//   then mbarriers                  full[slots], empty[slots]
template <int TF, int EPI, bool SHADOW>
__global__ void __launch_bounds__(kThreads, 2) linear_stream_kernel(const StreamParams sp) {
    constexpr int NT = TF / 8;  // n-tiles of 8 features
    const LinearParams& p = sp.base;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    const int x_stride = sp.in_padded + 8;  // bf16 elements per staged row (activations and weights)
    const int slot_bytes = TF * x_stride * 2;
    uint8_t* slot_base = smem;
    __nv_bfloat16* x_hi = reinterpret_cast<__nv_bfloat16*>(smem + sp.slots * slot_bytes);
    __nv_bfloat16* x_lo = x_hi + kRows * x_stride;
    float* partial = reinterpret_cast<float*>(x_lo + kRows * x_stride);
    uint64_t* full = reinterpret_cast<uint64_t*>(partial + kConsumers * kRows * TF);
    uint64_t* empty = full + sp.slots;
    uint64_t* xbar = empty + sp.slots;                                   // shadow input copies
    float* row_scale = reinterpret_cast<float*>(xbar + 1);               // [16]
    float* slices = row_scale + kRows;                                   // [16 slices][16 rows] sums of squares

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.y * kRows;
    const int my_tiles = (sp.tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

    // A bounded wait may run out in one consumer warp and not in another.  The warps therefore never leave on their own:
    // the one that gave up raises this flag, still arrives at the next barrier of the consumers, and all of them test the
    // flag behind that barrier and leave together.
    __shared__ int consumers_gave_up;
    if (threadIdx.x == 0) {
        for (int s = 0; s < sp.slots; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumers);
        }
        mbar_init(xbar, 1);
        consumers_gave_up = 0;
        mbar_fence_init();
    }
    // Columns in .. in_padded+8 of the weight slots are never written by the copies; the last k-step may read up to
    // 8 of them, so they are cleared once (stale bit patterns could be NaN, and 0 * NaN is NaN).
    if (p.in & 15) {
        for (int i = threadIdx.x; i < sp.slots * TF; i += kThreads) {
            __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(slot_base) + static_cast<size_t>(i) * x_stride;
            for (int k = p.in; k < x_stride; ++k) row[k] = __float2bfloat16_rn(0.0f);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores before async-proxy copies
    }
    __syncthreads();

    if (warp == kConsumers) {
        // ---- producer: lane i requests rows i, i+32, ... of every tile; lane 0 owns the barriers ----
        bool alive = true;
        for (int t = 0; t < my_tiles && alive; ++t) {
            const int tile = blockIdx.x + t * gridDim.x;
            const int s = t % sp.slots;
            const uint32_t phase = (t / sp.slots) & 1;
            int rows = p.out - tile * TF;
            if (rows > TF) rows = TF;
            if (lane == 0) {
                if (!mbar_wait(&empty[s], phase ^ 1)) {
                    atomicExch(sp.status, B200_DEVICE_TIMEOUT);
                    alive = false;
                } else {
                    mbar_expect_tx(&full[s], static_cast<uint32_t>(rows * p.in * 2));
                }
            }
            alive = __shfl_sync(0xffffffffu, alive, 0);
            if (!alive) break;
            const __nv_bfloat16* source = static_cast<const __nv_bfloat16*>(p.weight) + static_cast<int64_t>(tile) * TF * p.in;
            uint8_t* dst = slot_base + s * slot_bytes;
            for (int r = lane; r < rows; r += 32)
                bulk_load(dst + r * x_stride * 2, source + static_cast<int64_t>(r) * p.in, static_cast<uint32_t>(p.in * 2), &full[s]);
        }
        return;
    }

    // Weights are constants; the activations (and residual, cache, q) come from the preceding kernels.
    grid_dependency_wait();
    if constexpr (SHADOW) {
        // ---- consumers, shadow input: the rows arrive by bulk copy in their final form (one memory round trip, no
        // instructions); the row scales come from the producer's per-tile sums of squares.
        const int valid = p.rows - row0 < kRows ? p.rows - row0 : kRows;
        if (warp == 0) {
            if (lane == 0) mbar_expect_tx(xbar, static_cast<uint32_t>(2 * valid * p.in * 2));
            __syncwarp();
            const int r = lane & 15;
            if (r < valid) {
                const __nv_bfloat16* plane = lane < 16 ? p.x_hi : p.x_lo;
                bulk_load((lane < 16 ? x_hi : x_lo) + r * x_stride, plane + static_cast<int64_t>(row0 + r) * p.in,
                          static_cast<uint32_t>(p.in * 2), xbar);
            }
        }
        // Row scales: 16 threads per row-partial slice read the producer's per-tile sums of squares with independent
        // loads, the slices are added in a fixed order (deterministic), thread r finishes row r.
        {
            const int r = threadIdx.x & 15, slice = threadIdx.x >> 4;  // 16 slices of the partials
            float mine = 0.0f;
            if (p.sumsq_in && row0 + r < p.rows) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = slice + u * 16;
                    v[u] = i < p.parts_in ? __ldg(p.sumsq_in + static_cast<int64_t>(i) * p.rows + row0 + r) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) mine += v[u];
                for (int i = slice + 128; i < p.parts_in; i += 16) mine += __ldg(p.sumsq_in + static_cast<int64_t>(i) * p.rows + row0 + r);
            }
            slices[slice * kRows + r] = mine;
        }
        // The pad columns (in .. in_padded + 8) of all rows and the rows beyond the batch are zeros.
        {
            const int pad_words = (x_stride - p.in) >> 1;
            for (int i = threadIdx.x; i < 2 * kRows * pad_words; i += kConsumers * 32) {
                const int line = i / pad_words, word = i - line * pad_words;  // line = plane * 16 + row
                reinterpret_cast<uint32_t*>((line >= kRows ? x_lo : x_hi) + (line & (kRows - 1)) * x_stride + p.in)[word] = 0u;
            }
            const int row_words = p.in >> 1;
            for (int i = threadIdx.x; i < 2 * (kRows - valid) * row_words; i += kConsumers * 32) {
                const int line = i / row_words, word = i - line * row_words;
                const int plane = line / (kRows - valid), r = valid + line - plane * (kRows - valid);
                reinterpret_cast<uint32_t*>((plane ? x_lo : x_hi) + r * x_stride)[word] = 0u;
            }
        }
        if (!mbar_wait(xbar, 0)) {
            if (lane == 0) atomicExch(sp.status, B200_DEVICE_TIMEOUT);
            *static_cast<volatile int*>(&consumers_gave_up) = 1;
        }
        consumer_barrier();
        if (*static_cast<volatile int*>(&consumers_gave_up)) return;   // the activations never arrived: same decision in every consumer warp
        if (threadIdx.x < kRows) {  // read again only after the barrier that follows the first tile's products
            float scale = 1.0f;
            if (p.sumsq_in && row0 + threadIdx.x < p.rows) {
                float total = 0.0f;
#pragma unroll
                for (int slice = 0; slice < 16; ++slice) total += slices[slice * kRows + threadIdx.x];
                scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.in)), static_cast<float>(p.eps))));
            }
            row_scale[threadIdx.x] = scale;
        }
        // Only now may the successor start: its weight prefetch would otherwise queue ahead of the copies above.
        grid_launch_dependents();
    } else
    // ---- consumers: stage the activations (the weight stream is already in flight) ----
    // Warp w owns rows w and w+8.  Both rows are read with independent 16-byte loads into registers (one L2 round
    // trip), reduced to their RMS (f32 squares per lane, f64 across lanes and for the square root), normalised,
    // split into bf16 hi + lo and written to shared memory.  Rows longer than 1024 are handled one after the other.
    {
        const int vectors = p.in >> 2;             // float4 per row (in % 8 == 0)
        const int per_lane = (vectors + 31) >> 5;  // float4 per lane and row, at most 16
        auto stage_rows = [&](auto count_tag, int first_row) {
            constexpr int ROWS = decltype(count_tag)::value;  // rows handled together by this warp
            constexpr int MAXV = ROWS == 2 ? 8 : 16;
            float4 v[ROWS][MAXV];
#pragma unroll
            for (int q = 0; q < ROWS; ++q) {
                const int r = first_row + q * kConsumers;
                const bool valid = row0 + r < p.rows;
                const float4* source = reinterpret_cast<const float4*>(p.x + static_cast<int64_t>(valid ? row0 + r : 0) * p.in);
#pragma unroll
                for (int u = 0; u < MAXV; ++u) {
                    const int at = u * 32 + lane;
                    v[q][u] = (u < per_lane && valid && at < vectors) ? __ldg(source + at) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
#pragma unroll
            for (int q = 0; q < ROWS; ++q) {
                const int r = first_row + q * kConsumers;
                float scale = 1.0f;
                if (p.norm_weight) {
                    float squares = 0.0f;
#pragma unroll
                    for (int u = 0; u < MAXV; ++u)
                        if (u < per_lane) squares += v[q][u].x * v[q][u].x + v[q][u].y * v[q][u].y + v[q][u].z * v[q][u].z + v[q][u].w * v[q][u].w;
                    const float total = warp_sum(squares);
                    scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.in)), static_cast<float>(p.eps))));
                }
#pragma unroll
                for (int u = 0; u < MAXV; ++u) {
                    const int k = (u * 32 + lane) * 4;
                    if (u >= per_lane || k >= sp.in_padded) continue;
                    float e[4] = {v[q][u].x, v[q][u].y, v[q][u].z, v[q][u].w};
                    if (p.norm_weight && k < p.in) {
                        float w[4];
                        if (p.norm_dtype == B200_BF16) {
                            const uint2 packed = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.norm_weight) + k));
                            w[0] = bf16_lo(packed.x); w[1] = bf16_hi(packed.x); w[2] = bf16_lo(packed.y); w[3] = bf16_hi(packed.y);
                        } else {
                            const float4 f = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p.norm_weight) + k));
                            w[0] = f.x; w[1] = f.y; w[2] = f.z; w[3] = f.w;
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) e[i] = __fmul_rn(__fmul_rn(e[i], scale), w[i]);
                    }
                    const __nv_bfloat162 h0 = __floats2bfloat162_rn(e[0], e[1]), h1 = __floats2bfloat162_rn(e[2], e[3]);
                    const __nv_bfloat162 l0 = __floats2bfloat162_rn(e[0] - __low2float(h0), e[1] - __high2float(h0));
                    const __nv_bfloat162 l1 = __floats2bfloat162_rn(e[2] - __low2float(h1), e[3] - __high2float(h1));
                    uint2 hi, lo;
                    hi.x = *reinterpret_cast<const uint32_t*>(&h0); hi.y = *reinterpret_cast<const uint32_t*>(&h1);
                    lo.x = *reinterpret_cast<const uint32_t*>(&l0); lo.y = *reinterpret_cast<const uint32_t*>(&l1);
                    *reinterpret_cast<uint2*>(x_hi + r * x_stride + k) = hi;
                    *reinterpret_cast<uint2*>(x_lo + r * x_stride + k) = lo;
                }
            }
        };
        // in_padded beyond in: the tail columns of a row are written as zeros by the lanes that own them
        if (per_lane <= 8) {
            stage_rows(std::integral_constant<int, 2>{}, warp);
        } else {
            stage_rows(std::integral_constant<int, 1>{}, warp);
            stage_rows(std::integral_constant<int, 1>{}, warp + kConsumers);
        }
        consumer_barrier();
        grid_launch_dependents();
    }

    const int mi = lane >> 3, ri = lane & 7;
    // ldmatrix row address of the activation fragment: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
    const uint32_t a_lane = static_cast<uint32_t>((((mi & 1) * 8 + ri) * x_stride + (mi >> 1) * 8) * 2);
    const uint32_t a_hi = smem_u32(x_hi) + a_lane, a_lo = smem_u32(x_lo) + a_lane;
    const int ksteps = (p.in + 15) >> 4;

    // B200_EPI_ARGMAX: the row candidates this thread has seen over the CTA's tiles (one per pass of the finishing loop)
    Candidate running[TF > 32 ? 2 : 1];
#pragma unroll
    for (int i = 0; i < (TF > 32 ? 2 : 1); ++i) running[i] = Candidate{-INFINITY, INT32_MAX};

    bool alive = true;
    for (int t = 0; t < my_tiles && alive; ++t) {
        const int tile = blockIdx.x + t * gridDim.x;
        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
        // The residual values this thread will add in the tile's epilogue are requested now, under the products.
        float2 carried = make_float2(0.0f, 0.0f);
        if constexpr (SHADOW && EPI == B200_EPI_RESIDUAL && TF <= 32) {
            const int r = threadIdx.x / (TF / 2), f = (threadIdx.x - r * (TF / 2)) * 2;
            const int row = row0 + r, feature0 = tile * TF + f;
            if (r < kRows && row < p.rows && feature0 + 1 < p.out)
                carried = *reinterpret_cast<const float2*>(p.residual + static_cast<int64_t>(row) * p.out + feature0);
        }
        {
            const int s = t % sp.slots;
            const uint32_t phase = (t / sp.slots) & 1;
            if (!mbar_wait(&full[s], phase)) {
                if (lane == 0) atomicExch(sp.status, B200_DEVICE_TIMEOUT);
                *static_cast<volatile int*>(&consumers_gave_up) = 1;
                alive = false;
            }
            const uint32_t slot = smem_u32(slot_base + s * slot_bytes);
            // ldmatrix row addresses of the weight fragments: x4 = (features n*8.., k 0-7), (same, k 8-15),
            // (features (n+1)*8.., k 0-7), (same, k 8-15); x2 = the first two
            const uint32_t b_lane = slot + static_cast<uint32_t>((((NT == 1 ? 0 : (mi >> 1)) * 8 + ri) * x_stride + (mi & 1) * 8) * 2);
            for (int j = warp; alive && j < ksteps; j += kConsumers) {
                uint32_t ah[4], al[4];
                const uint32_t column_bytes = static_cast<uint32_t>(j * 32);
                ldmatrix_x4(ah, a_hi + column_bytes);
                ldmatrix_x4(al, a_lo + column_bytes);
                if constexpr (NT == 1) {
                    uint32_t b[2];
                    ldmatrix_x2(b, b_lane + column_bytes);
                    mma_bf16(acc[0], ah, b[0], b[1]);
                    mma_bf16(acc[0], al, b[0], b[1]);
                } else {
#pragma unroll
                    for (int n = 0; n < NT; n += 2) {
                        uint32_t b[4];
                        ldmatrix_x4(b, b_lane + static_cast<uint32_t>(n * 8 * x_stride * 2) + column_bytes);
                        mma_bf16(acc[n], ah, b[0], b[1]);
                        mma_bf16(acc[n], al, b[0], b[1]);
                        mma_bf16(acc[n + 1], ah, b[2], b[3]);
                        mma_bf16(acc[n + 1], al, b[2], b[3]);
                    }
                }
            }
            __syncwarp();
            if (alive && lane == 0) mbar_arrive(&empty[s]);
        }
        // ---- add the eight K-slices and finish the tile ----
        {
            const int g = lane >> 2, tq = lane & 3;
            float* mine = partial + warp * kRows * TF;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                *reinterpret_cast<float2*>(mine + g * TF + n * 8 + 2 * tq) = make_float2(acc[n][0], acc[n][1]);
                *reinterpret_cast<float2*>(mine + (g + 8) * TF + n * 8 + 2 * tq) = make_float2(acc[n][2], acc[n][3]);
            }
        }
        consumer_barrier();
        if (*static_cast<volatile int*>(&consumers_gave_up)) break;   // a weight tile never arrived: every consumer warp leaves here
        // items of one row are TF/2 consecutive threads of a warp: thread i finishes the feature pair (r, f)
#pragma unroll
        for (int base = 0; base < kRows * (TF / 2); base += kConsumers * 32) {
            const int i = base + threadIdx.x;
            const int r = i / (TF / 2), f = (i - r * (TF / 2)) * 2;
            const bool in_tile = i < kRows * (TF / 2);
            float a = 0.0f, b = 0.0f;
            if (in_tile) {
#pragma unroll
                for (int w = 0; w < kConsumers; ++w) {
                    const float2 v = *reinterpret_cast<const float2*>(partial + (w * kRows + r) * TF + f);
                    a += v.x;
                    b += v.y;
                }
            }
            const int row = row0 + r, feature0 = tile * TF + f;
            const bool live = in_tile && row < p.rows && feature0 < p.out;
            if constexpr (SHADOW) {
                if (in_tile) { a *= row_scale[r]; b *= row_scale[r]; }
            }
            if constexpr (SHADOW && EPI == B200_EPI_RESIDUAL && TF <= 32) {
                if (live) {  // out is even on the shadow path, so the pair is complete
                    a = __fadd_rn(carried.x, a);
                    b = __fadd_rn(carried.y, b);
                    *reinterpret_cast<float2*>(p.y + static_cast<int64_t>(row) * p.out + feature0) = make_float2(a, b);
                    store_copies(p, static_cast<int64_t>(row) * p.out + feature0, a, b, true);
                }
            } else {
                if (live) linear_epilogue<EPI>(p, row, feature0, a, b);
            }
            if constexpr (SHADOW && EPI == B200_EPI_RESIDUAL) {
                // a, b now hold the new residual-stream values: shadow for the consumer, row sums of squares for its norm
                float square = live ? a * a + (feature0 + 1 < p.out ? b * b : 0.0f) : 0.0f;
#pragma unroll
                for (int o = 1; o < TF / 2; o <<= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
                if (p.sumsq_out && f == 0 && in_tile && row < p.rows) p.sumsq_out[static_cast<int64_t>(tile) * p.rows + row] = square;
                if (p.out_hi && live) {
                    float wa = 1.0f, wb = 1.0f;
                    if (p.out_norm_weight) {
                        const bool second = feature0 + 1 < p.out;
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
                    const int64_t at = static_cast<int64_t>(row) * p.out + feature0;  // out is even on this path
                    *reinterpret_cast<__nv_bfloat162*>(p.out_hi + at) = hi;
                    *reinterpret_cast<__nv_bfloat162*>(p.out_lo + at) = lo;
                }
            }
            if constexpr (EPI == B200_EPI_ARGMAX) {
                // the TF/2 threads of a row are consecutive lanes: butterfly to the row's candidate of this tile
                Candidate best = live ? pair_candidate(feature0, a, b, p.out) : Candidate{-INFINITY, INT32_MAX};
#pragma unroll
                for (int o = 1; o < TF / 2; o <<= 1) {
                    const Candidate other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
                    if (preferred(other, best)) best = other;
                }
                if (preferred(best, running[base / (kConsumers * 32)])) running[base / (kConsumers * 32)] = best;
            }
            if constexpr (SHADOW && EPI == B200_EPI_SWIGLU) {
                if (p.out_hi && live) {
                    const __nv_bfloat16 hi = __float2bfloat16_rn(a);
                    const int64_t at = static_cast<int64_t>(row) * (p.out >> 1) + (feature0 >> 1);
                    p.out_hi[at] = hi;
                    p.out_lo[at] = __float2bfloat16_rn(a - __bfloat162float(hi));
                }
            }
        }
        consumer_barrier();
    }
    if constexpr (EPI == B200_EPI_ARGMAX) {
        // one candidate per row and CTA: thread (row r, first pair) holds the best of the CTA's tiles
#pragma unroll
        for (int base = 0; base < kRows * (TF / 2); base += kConsumers * 32) {
            const int i = base + threadIdx.x;
            const int r = i / (TF / 2), f = i - r * (TF / 2);
            if (alive && f == 0 && i < kRows * (TF / 2) && row0 + r < p.rows) {
                p.best_value[static_cast<int64_t>(blockIdx.x) * p.rows + row0 + r] = running[base / (kConsumers * 32)].value;
                p.best_index[static_cast<int64_t>(blockIdx.x) * p.rows + row0 + r] = running[base / (kConsumers * 32)].index;
            }
        }
    }
}

template <int TF, int EPI, bool SHADOW> int launch_mode(const StreamParams& sp, size_t smem, int ctas, int row_tiles, cudaStream_t stream) {
    auto kernel = linear_stream_kernel<TF, EPI, SHADOW>;
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    return cuda_status(launch_dependent(kernel, dim3(ctas, row_tiles), dim3(kThreads), smem, stream, sp), "linear_stream_kernel launch");
}

template <int TF, int EPI> int launch_tile(const StreamParams& sp, size_t smem, int ctas, int row_tiles, cudaStream_t stream) {
    return sp.base.x_hi ? launch_mode<TF, EPI, true>(sp, smem, ctas, row_tiles, stream)
                        : launch_mode<TF, EPI, false>(sp, smem, ctas, row_tiles, stream);
}

template <int EPI> int pick_tile(const StreamParams& sp, size_t smem, int ctas, int row_tiles, cudaStream_t stream) {
    switch (sp.tile_features) {
    case 8: return launch_tile<8, EPI>(sp, smem, ctas, row_tiles, stream);
    case 16: return launch_tile<16, EPI>(sp, smem, ctas, row_tiles, stream);
    case 32: return launch_tile<32, EPI>(sp, smem, ctas, row_tiles, stream);
    default: return launch_tile<64, EPI>(sp, smem, ctas, row_tiles, stream);
    }
}

// Tile size, ring depth and shared-memory size for a weight matrix [out, in]; false when nothing fits.
bool choose_tiling(int in, int out, int sms, StreamParams& sp, size_t& smem) {
    sp.in_padded = (in + 63) & ~63;
    const size_t row_bytes = static_cast<size_t>(sp.in_padded + 8) * 2;
    // Smallest tile with which one round of CTAs covers the matrix (every further tile of a CTA costs a reduction
    // round).  Half of the shared memory is preferred (two CTAs per SM: this kernel's tail next to the early-started
    // successor), the whole when a ring of two tiles does not fit in half, a smaller tile when it does not fit at all.
    const size_t half = 110 * 1024, whole = 220 * 1024;
    int tf = 8;
    while (tf < 64 && (out + tf - 1) / tf > sms) tf <<= 1;
    size_t fixed = 0;
    int slots = 0;
    for (;; tf >>= 1) {
        fixed = 2 * kRows * row_bytes + static_cast<size_t>(kConsumers) * kRows * tf * 4 + 128 + 1536;
        slots = fixed < half ? static_cast<int>((half - fixed) / (tf * row_bytes)) : 0;
        if (slots < 2) slots = fixed < whole ? static_cast<int>((whole - fixed) / (tf * row_bytes)) : 0;
        if (slots >= 2 || tf == 8) break;
    }
    if (slots < 2) return false;
    if (slots > 8) slots = 8;
    sp.tile_features = tf;
    sp.slots = slots;
    sp.tiles = (out + tf - 1) / tf;
    smem = fixed + static_cast<size_t>(slots) * tf * row_bytes;
    return true;
}

}  // namespace

int linear_stream_parts(int rows, int in, int out) {
    if ((in & 7) || in <= 0 || out <= 0) return 0;
    if (rows >= kGemmRows || in > kMaxIn) return linear_gemm_parts(rows, in, out);
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); device = -1; }   // no device: the figures of a 148-SM part
    StreamParams sp{};
    size_t smem = 0;
    return choose_tiling(in, out, sm_count(device), sp, smem) ? sp.tiles : 0;
}

int linear_argmax_parts(int rows, int in, int out) {
    if ((in & 7) || in <= 0 || out <= 0) return 0;
    if (rows >= kGemmRows || in > kMaxIn) return linear_gemm_parts(rows, in, out);
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); device = -1; }
    StreamParams sp{};
    size_t smem = 0;
    if (!choose_tiling(in, out, sm_count(device), sp, smem)) return 0;
    return sp.tiles < sm_count(device) ? sp.tiles : sm_count(device);   // one candidate slice per CTA
}

// ---- thin outputs (adapter down-projections: a few dozen output features) for passes the dense kernel would serve ----
// A 128-wide tensor-core tile would be one mostly empty tile with a K split of four CTAs at the kernel's latency floor.
// Here a CTA takes one activation row and eight output features: 256 threads stride over K with 16-byte loads (eight
// activation values from the hi (+ lo) planes, eight weights per feature), f32 FMAs, then a block reduction.  The
// operands are a few hundred KB that every CTA finds in L2.
constexpr int kThinFeatures = 8, kThinThreads = 256, kThinMaxOut = 64;

__global__ void __launch_bounds__(kThinThreads) linear_thin_kernel(const LinearParams p) {
    __shared__ float partial[kThinThreads / 32][kThinFeatures];
    grid_dependency_wait();
    grid_launch_dependents();
    const int row = blockIdx.x, feature0 = blockIdx.y * kThinFeatures;
    const auto* weight = static_cast<const __nv_bfloat16*>(p.weight);
    float acc[kThinFeatures];
#pragma unroll
    for (int f = 0; f < kThinFeatures; ++f) acc[f] = 0.0f;
    for (int k = threadIdx.x * 8; k < p.in; k += kThinThreads * 8) {
        const uint4 hi = *reinterpret_cast<const uint4*>(p.x_hi + static_cast<int64_t>(row) * p.in + k);
        uint4 lo = make_uint4(0u, 0u, 0u, 0u);
        if (p.x_lo) lo = *reinterpret_cast<const uint4*>(p.x_lo + static_cast<int64_t>(row) * p.in + k);
        const uint32_t h[4] = {hi.x, hi.y, hi.z, hi.w}, l[4] = {lo.x, lo.y, lo.z, lo.w};
        float x[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = bf16_lo(h[i]) + bf16_lo(l[i]);
            x[2 * i + 1] = bf16_hi(h[i]) + bf16_hi(l[i]);
        }
#pragma unroll
        for (int f = 0; f < kThinFeatures; ++f) {
            if (feature0 + f >= p.out) break;
            const uint4 w = __ldg(reinterpret_cast<const uint4*>(weight + static_cast<int64_t>(feature0 + f) * p.in + k));
            const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[f] = fmaf(x[2 * i], bf16_lo(v[i]), fmaf(x[2 * i + 1], bf16_hi(v[i]), acc[f]));
        }
    }
#pragma unroll
    for (int f = 0; f < kThinFeatures; ++f) acc[f] = warp_sum(acc[f]);
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int f = 0; f < kThinFeatures; ++f) partial[threadIdx.x >> 5][f] = acc[f];
    }
    __syncthreads();
    if (threadIdx.x < kThinFeatures && feature0 + threadIdx.x < p.out) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kThinThreads / 32; ++w) total += partial[w][threadIdx.x];
        float scale = 1.0f;
        if (p.sumsq_in) {
            float squares = 0.0f;
            for (int i = 0; i < p.parts_in; ++i) squares += __ldg(p.sumsq_in + static_cast<int64_t>(i) * p.rows + row);
            scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, static_cast<float>(p.in)), static_cast<float>(p.eps))));
        }
        p.y[static_cast<int64_t>(row) * p.out + feature0 + threadIdx.x] = total * scale;
    }
}

int launch_linear_thin(const LinearParams& p, cudaStream_t stream) {
    const dim3 grid(static_cast<unsigned>(p.rows), static_cast<unsigned>((p.out + kThinFeatures - 1) / kThinFeatures));
    return cuda_status(launch_dependent(linear_thin_kernel, grid, dim3(kThinThreads), 0, stream, p), "linear_thin_kernel launch");
}

int launch_linear_stream(const LinearParams& p, int epilogue, cudaStream_t stream) {
    if (p.x_hi && (p.rows >= kGemmRows || p.in > kMaxIn) && epilogue == B200_EPI_STORE && p.out <= kThinMaxOut && p.rows <= 512
        && p.weight_dtype == B200_BF16 && (p.in & 7) == 0
        && ((reinterpret_cast<uintptr_t>(p.weight) | reinterpret_cast<uintptr_t>(p.x_hi) | reinterpret_cast<uintptr_t>(p.x_lo)) & 15) == 0)
        return launch_linear_thin(p, stream);
    if (p.x_hi && (p.rows >= kGemmRows || p.in > kMaxIn)) return launch_linear_gemm(p, epilogue, stream);
    if (p.x_hi && !p.x_lo) return B200_UNSUPPORTED;   // the streaming kernel always multiplies both planes
    if (p.weight_dtype != B200_BF16 || p.in > kMaxIn || (p.in & 7) || (reinterpret_cast<uintptr_t>(p.weight) & 15))
        return B200_UNSUPPORTED;
    if (p.x_hi ? ((reinterpret_cast<uintptr_t>(p.x_hi) | reinterpret_cast<uintptr_t>(p.x_lo)) & 15) || !p.x_lo
               : (reinterpret_cast<uintptr_t>(p.x) & 15) != 0)
        return B200_UNSUPPORTED;
    if (p.out_hi && (p.out & 1)) return B200_UNSUPPORTED;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    const int sms = sm_count(device);

    StreamParams sp{};
    sp.base = p;
    sp.status = device_status_word(device);
    if (!sp.status) { set_error("the device status word could not be allocated"); return B200_NO_DEVICE; }
    size_t smem = 0;
    if (!choose_tiling(p.in, p.out, sms, sp, smem)) return B200_UNSUPPORTED;

    const int row_tiles = (p.rows + kRows - 1) / kRows;
    const int ctas = sp.tiles < sms ? sp.tiles : sms;
    switch (epilogue) {
    case B200_EPI_STORE: return pick_tile<B200_EPI_STORE>(sp, smem, ctas, row_tiles, stream);
    case B200_EPI_RESIDUAL: return pick_tile<B200_EPI_RESIDUAL>(sp, smem, ctas, row_tiles, stream);
    case B200_EPI_SWIGLU: return pick_tile<B200_EPI_SWIGLU>(sp, smem, ctas, row_tiles, stream);
    case B200_EPI_QKV: return pick_tile<B200_EPI_QKV>(sp, smem, ctas, row_tiles, stream);
    case B200_EPI_ARGMAX: return p.x_hi ? pick_tile<B200_EPI_ARGMAX>(sp, smem, ctas, row_tiles, stream) : B200_UNSUPPORTED;
    }
    return B200_UNSUPPORTED;
}

}  // namespace b200

