// Row-wise finishing of an accumulator tile held row-major in shared memory: shared by the dense kernels.
#pragma once

#include "linear_common.cuh"

namespace b200 {

// q|k|v epilogue: where the token of activation row `row` goes - its position (cache length + offset inside the chunk) and
// the physical page of that position - looked up once per row instead of once per feature pair.
__device__ __forceinline__ int2 qkv_row_place(const LinearParams& p, int row) {
    if (row >= p.rows) return make_int2(0, 0);
    const int sequence = row / p.tokens_per_sequence;
    const int position = __ldg(p.kv.lengths + sequence) + row % p.tokens_per_sequence;
    int page_slot = position / p.kv.page_size;
    if (page_slot >= p.kv.pages_per_seq) page_slot = p.kv.pages_per_seq - 1;
    return make_int2(position, __ldg(p.kv.page_table + static_cast<int64_t>(sequence) * p.kv.pages_per_seq + page_slot));
}

// One finished pair of adjacent features of one token row: shared epilogue, then the optional output shadow (hi + lo of
// the value times the next norm weight) and the running sum of squares of the new residual stream.
// `carried` holds the residual values of the pair (B200_EPI_RESIDUAL only), loaded ahead by the caller.
template <int EPI>
__device__ __forceinline__ void finish_pair(const LinearParams& p, int row, int feature0, float a, float b, float2 carried, float& squares,
                                            const int2* place = nullptr) {
    if constexpr (EPI == B200_EPI_RESIDUAL) {
        const bool second = feature0 + 1 < p.out;
        const int64_t at = static_cast<int64_t>(row) * p.out + feature0;
        a = __fadd_rn(carried.x, a);
        b = second ? __fadd_rn(carried.y, b) : 0.0f;
        if ((p.out & 1) == 0) {
            *reinterpret_cast<float2*>(p.y + at) = make_float2(a, b);
        } else {
            p.y[at] = a;
            if (second) p.y[at + 1] = b;
        }
        store_copies(p, at, a, b, second);
    } else {
        linear_epilogue<EPI>(p, row, feature0, a, b, place);
    }
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

// Finishes the rows [first, last) of a tile held row-major in shared memory (`tile`, or the sum over the cluster's
// `split` partial tiles `peer_tile[z]`).  Warp `worker` of `workers` takes kBatch consecutive rows per iteration: first
// every value the rows need is requested (accumulators from shared memory or from the peers, residual pairs from global
// memory), then the rows are finished, so the memory round trips of the rows overlap instead of queueing behind each
// other.  Lanes run across the feature pairs: every global access is coalesced; per-row reductions are butterflies.
template <int EPI, int kTileN>
__device__ __forceinline__ void finish_rows(const LinearParams& p, const float* tile, const uint32_t (&peer_tile)[8], int split,
                                            const float* row_scale, int m0, int n0, int feature_tile, int first, int last, int worker,
                                            int workers, int lane, bool ready, const int2* row_place = nullptr) {
    constexpr int kTileStride = kTileN + 4;
        constexpr int kBatch = 4, kPasses = kTileN / 64;
        for (int base = first + worker * kBatch; base < last; base += workers * kBatch) {
            float2 value[kBatch][kPasses], carried[kBatch][kPasses];
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
                const int tile_row = base + r, row = m0 + tile_row;
                const bool live_row = tile_row < last && row < p.rows;
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    const int c = pass * 64 + lane * 2;
                    const int feature0 = n0 + c;
                    value[r][pass] = make_float2(0.0f, 0.0f);
                    carried[r][pass] = make_float2(0.0f, 0.0f);
                    if (!live_row) continue;
                    if (split == 1) {
                        value[r][pass] = *reinterpret_cast<const float2*>(tile + tile_row * kTileStride + c);
                    } else {
                        const uint32_t offset = static_cast<uint32_t>(tile_row * kTileStride + c) * 4;
                        float2 v[8];
#pragma unroll
                        for (int z = 0; z < 8; ++z) v[z] = z < split ? load_cluster_float2(peer_tile[z] + offset) : make_float2(0.0f, 0.0f);
                        float2 sum = v[0];
#pragma unroll
                        for (int z = 1; z < 8; ++z) { sum.x += v[z].x; sum.y += v[z].y; }
                        value[r][pass] = sum;
                    }
                    if constexpr (EPI == B200_EPI_RESIDUAL) {
                        if (feature0 < p.out) {
                            const float* source = p.residual + static_cast<int64_t>(row) * p.out + feature0;
                            if ((p.out & 1) == 0) carried[r][pass] = *reinterpret_cast<const float2*>(source);
                            else carried[r][pass] = make_float2(source[0], feature0 + 1 < p.out ? source[1] : 0.0f);
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
                const int tile_row = base + r, row = m0 + tile_row;
                if (tile_row >= last || row >= p.rows) break;
                const float scale = row_scale[tile_row];
                float squares = 0.0f;
                Candidate best{-INFINITY, INT32_MAX};
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    const int feature0 = n0 + pass * 64 + lane * 2;
                    if (!ready || feature0 >= p.out) continue;
                    const float a = value[r][pass].x * scale, b = value[r][pass].y * scale;
                    if constexpr (EPI == B200_EPI_ARGMAX) {
                        const Candidate pair = pair_candidate(feature0, a, b, p.out);
                        if (preferred(pair, best)) best = pair;
                    } else {
                        finish_pair<EPI>(p, row, feature0, a, b, carried[r][pass], squares, row_place ? row_place + tile_row : nullptr);
                    }
                }
                if constexpr (EPI == B200_EPI_RESIDUAL) {
                    if (p.sumsq_out) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, o);
                        if (lane == 0) p.sumsq_out[static_cast<int64_t>(feature_tile) * p.rows + row] = squares;
                    }
                }
                if constexpr (EPI == B200_EPI_ARGMAX) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const Candidate other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
                        if (preferred(other, best)) best = other;
                    }
                    if (lane == 0) {
                        p.best_value[static_cast<int64_t>(feature_tile) * p.rows + row] = best.value;
                        p.best_index[static_cast<int64_t>(feature_tile) * p.rows + row] = best.index;
                    }
                }
            }
        }
    }

}  // namespace b200
