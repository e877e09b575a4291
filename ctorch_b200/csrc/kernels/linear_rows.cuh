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

// Whether the vector form applies to this call: every matrix the epilogue touches is addressed in 16-byte (f32) or
// 8-byte (bf16 shadow) units per lane.  The greedy-choice epilogue stores nothing and always qualifies.
template <int EPI>
__host__ __device__ __forceinline__ bool rows_take_quads(const LinearParams& p) {
    if constexpr (EPI == B200_EPI_ARGMAX) return true;
    if (p.out & 3) return false;
    uintptr_t bits = 0;
    if constexpr (EPI == B200_EPI_STORE || EPI == B200_EPI_RESIDUAL) {
        bits |= reinterpret_cast<uintptr_t>(p.y);
        if (p.copies > 0) bits |= reinterpret_cast<uintptr_t>(p.y_copy[0]);
        if (p.copies > 1) bits |= reinterpret_cast<uintptr_t>(p.y_copy[1]);
        if (p.copies > 2) bits |= reinterpret_cast<uintptr_t>(p.y_copy[2]);
        if (p.copies > 3) bits |= reinterpret_cast<uintptr_t>(p.y_copy[3]);
        if (p.copies > 4) bits |= reinterpret_cast<uintptr_t>(p.y_copy[4]);
        if (p.copies > 5) bits |= reinterpret_cast<uintptr_t>(p.y_copy[5]);
        if (p.copies > 6) bits |= reinterpret_cast<uintptr_t>(p.y_copy[6]);
    }
    if constexpr (EPI == B200_EPI_RESIDUAL) {
        bits |= reinterpret_cast<uintptr_t>(p.residual) | (reinterpret_cast<uintptr_t>(p.out_hi) << 1) | (reinterpret_cast<uintptr_t>(p.out_lo) << 1)
              | (p.out_norm_dtype == B200_BF16 ? reinterpret_cast<uintptr_t>(p.out_norm_weight) << 1 : reinterpret_cast<uintptr_t>(p.out_norm_weight));
    }
    if constexpr (EPI == B200_EPI_SWIGLU)
        bits |= (reinterpret_cast<uintptr_t>(p.y) << 1) | (reinterpret_cast<uintptr_t>(p.out_hi) << 2) | (reinterpret_cast<uintptr_t>(p.out_lo) << 2);
    if constexpr (EPI == B200_EPI_QKV) {
        if (p.head_dim & 3) return false;   // a quad never straddles q | k | v or two heads
        bits |= reinterpret_cast<uintptr_t>(p.q_out) | reinterpret_cast<uintptr_t>(p.cosine) << 1 | reinterpret_cast<uintptr_t>(p.sine) << 1
              | reinterpret_cast<uintptr_t>(p.kv.pool[0]) | reinterpret_cast<uintptr_t>(p.kv.pool[1]);
    }
    return (bits & 15) == 0;
}

// The same from this CTA's own shared memory (an address of the CTA's window): the plain path, which does not go through
// the cluster's network.
__device__ __forceinline__ float4 load_shared_float4(uint32_t address) {
    float4 value;
    asm("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(value.x), "=f"(value.y), "=f"(value.z), "=f"(value.w) : "r"(address));
    return value;
}
__device__ __forceinline__ float4 load_cluster_float4(uint32_t cluster_address) {
    float4 value;
    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(value.x), "=f"(value.y), "=f"(value.z), "=f"(value.w) : "r"(cluster_address));
    return value;
}

// Residual values of kBatch rows (rows past `last` repeat the last one), four features per lane and pass.
template <int EPI, int kBatch, int kPasses>
__device__ __forceinline__ void fetch_residual_quads(const LinearParams& p, int m0, int n0, int last, int lane, int base,
                                                     float4 (&into)[kBatch][kPasses]) {
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
        const int row = m0 + min(base + r, last - 1);
#pragma unroll
        for (int pass = 0; pass < kPasses; ++pass) {
            into[r][pass] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if constexpr (EPI == B200_EPI_RESIDUAL) {
                const int feature0 = n0 + pass * 128 + lane * 4;
                if (feature0 < p.out) into[r][pass] = *reinterpret_cast<const float4*>(p.residual + static_cast<int64_t>(row) * p.out + feature0);
            }
        }
    }
}

// Vector form of finish_rows_pairs below: a lane holds four adjacent features, so a 128-feature row is one instruction
// per access.  A batch of kBatch rows is worked in three straight-line phases - fetch (accumulators, residual values),
// arithmetic, stores - with no branch between the rows, so that the rows' dependent chains (shared-memory load, scale,
// exponential, reciprocal, roundings) overlap: with twelve warps on an SM nothing else hides those latencies.  Rows past
// the end repeat the last live row (the same values go to the same places twice) instead of being branched around.
template <int EPI, int kTileN, bool kLocal>
__device__ __forceinline__ void finish_rows_quads(const LinearParams& p, const float* tile, const uint32_t (&peer_tile)[8], int split,
                                                  const float* row_scale, int m0, int n0, int feature_tile, int first, int last, int worker,
                                                  int workers, int lane, bool ready, const int2* row_place) {
    constexpr int kTileStride = kTileN + 4;
    constexpr int kBatch = 4, kPasses = kTileN / 128;
    if (last > p.rows - m0) last = p.rows - m0;
    if (first >= last) return;
    float4 norm[kPasses];
    bool live[kPasses];   // this lane's four features exist and the accumulators are valid
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
        const int feature0 = n0 + pass * 128 + lane * 4;
        live[pass] = ready && feature0 < p.out;
        norm[pass] = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        if constexpr (EPI == B200_EPI_RESIDUAL) {
            if (p.out_hi && p.out_norm_weight && feature0 < p.out) {
                if (p.out_norm_dtype == B200_BF16) {
                    const uint2 w = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.out_norm_weight) + feature0));
                    norm[pass] = make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                                             __uint_as_float(w.y & 0xffff0000u));
                } else {
                    norm[pass] = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p.out_norm_weight) + feature0));
                }
            }
        }
    }
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    // q | k | v: what a lane's four features are does not depend on the row - region, head and offset inside the head
    // (a quad never straddles q | k | v or a head: rows_take_quads)
    int region[kPasses], local[kPasses], head[kPasses], inside[kPasses];
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
        region[pass] = 0; local[pass] = 0; head[pass] = 0; inside[pass] = 0;
        if constexpr (EPI == B200_EPI_QKV) {
            const int D = p.heads * p.head_dim, KV = p.kv_heads * p.head_dim;
            int l = n0 + pass * 128 + lane * 4;
            if (l >= D) { region[pass] = 1; l -= D; }
            if (region[pass] == 1 && l >= KV) { region[pass] = 2; l -= KV; }
            local[pass] = l;
            head[pass] = l / p.head_dim;
            inside[pass] = l - head[pass] * p.head_dim;
        }
    }
    float4 carried[kBatch][kPasses];
    int base = first + worker * kBatch;
    if (base < last) fetch_residual_quads<EPI, kBatch, kPasses>(p, m0, n0, last, lane, base, carried);
    for (; base < last; base += workers * kBatch) {
        float4 value[kBatch][kPasses], ahead[kBatch][kPasses];
        int rows[kBatch];
        float scale[kBatch];
        // ---- fetch ----
#pragma unroll
        for (int r = 0; r < kBatch; ++r) {
            const int tile_row = min(base + r, last - 1);
            rows[r] = tile_row;
            scale[r] = row_scale[tile_row];
#pragma unroll
            for (int pass = 0; pass < kPasses; ++pass) {
                const int c = pass * 128 + lane * 4;
                if (split == 1) {
                    value[r][pass] = *reinterpret_cast<const float4*>(tile + tile_row * kTileStride + c);
                } else {
                    const uint32_t offset = static_cast<uint32_t>(tile_row * kTileStride + c) * 4;
                    float4 v[8];
#pragma unroll
                    for (int z = 0; z < 8; ++z) v[z] = z < split ? (kLocal ? load_shared_float4(peer_tile[z] + offset) : load_cluster_float4(peer_tile[z] + offset)) : zero;
                    float4 sum = v[0];
#pragma unroll
                    for (int z = 1; z < 8; ++z) { sum.x += v[z].x; sum.y += v[z].y; sum.z += v[z].z; sum.w += v[z].w; }
                    value[r][pass] = sum;
                }
            }
        }
        if constexpr (EPI == B200_EPI_RESIDUAL) {
            if (base + workers * kBatch < last) fetch_residual_quads<EPI, kBatch, kPasses>(p, m0, n0, last, lane, base + workers * kBatch, ahead);
        }
        // ---- arithmetic (no branches) and stores ----
        if constexpr (EPI == B200_EPI_RESIDUAL) {
            float4 sum[kBatch][kPasses];
            uint2 hi[kBatch][kPasses], lo[kBatch][kPasses];
            float squares[kBatch];
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
                squares[r] = 0.0f;
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    const float4 v = value[r][pass], c = carried[r][pass];
                    float4 t = make_float4(__fadd_rn(c.x, v.x * scale[r]), __fadd_rn(c.y, v.y * scale[r]), __fadd_rn(c.z, v.z * scale[r]),
                                           __fadd_rn(c.w, v.w * scale[r]));
                    if (!live[pass]) t = zero;
                    sum[r][pass] = t;
                    squares[r] += t.x * t.x + t.y * t.y;
                    squares[r] += t.z * t.z + t.w * t.w;
                    const float a = __fmul_rn(t.x, norm[pass].x), b = __fmul_rn(t.y, norm[pass].y), c2 = __fmul_rn(t.z, norm[pass].z),
                                d = __fmul_rn(t.w, norm[pass].w);
                    const __nv_bfloat162 hi0 = __floats2bfloat162_rn(a, b), hi1 = __floats2bfloat162_rn(c2, d);
                    const __nv_bfloat162 lo0 = __floats2bfloat162_rn(a - __low2float(hi0), b - __high2float(hi0));
                    const __nv_bfloat162 lo1 = __floats2bfloat162_rn(c2 - __low2float(hi1), d - __high2float(hi1));
                    hi[r][pass] = make_uint2(*reinterpret_cast<const uint32_t*>(&hi0), *reinterpret_cast<const uint32_t*>(&hi1));
                    lo[r][pass] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo0), *reinterpret_cast<const uint32_t*>(&lo1));
                }
            }
            if (p.sumsq_out && ready) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                    for (int r = 0; r < kBatch; ++r) squares[r] += __shfl_xor_sync(0xffffffffu, squares[r], o);
                }
                if (lane < kBatch) {
                    float mine = squares[0];
#pragma unroll
                    for (int r = 1; r < kBatch; ++r) mine = lane == r ? squares[r] : mine;
                    int row_of_lane = rows[0];
#pragma unroll
                    for (int r = 1; r < kBatch; ++r) row_of_lane = lane == r ? rows[r] : row_of_lane;
                    p.sumsq_out[static_cast<int64_t>(feature_tile) * p.rows + m0 + row_of_lane] = mine;
                }
            }
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    if (!live[pass]) continue;
                    const int64_t at = static_cast<int64_t>(m0 + rows[r]) * p.out + n0 + pass * 128 + lane * 4;
                    *reinterpret_cast<float4*>(p.y + at) = sum[r][pass];
                    if (p.out_hi) {
                        *reinterpret_cast<uint2*>(p.out_hi + at) = hi[r][pass];
                        *reinterpret_cast<uint2*>(p.out_lo + at) = lo[r][pass];
                    }
                }
            }
            if (p.copies > 0) {
#pragma unroll
                for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                    for (int pass = 0; pass < kPasses; ++pass) {
                        if (!live[pass]) continue;
                        const int64_t at = static_cast<int64_t>(m0 + rows[r]) * p.out + n0 + pass * 128 + lane * 4;
                        store_copies(p, at, sum[r][pass]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kBatch; ++r)
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) carried[r][pass] = ahead[r][pass];
        } else if constexpr (EPI == B200_EPI_SWIGLU) {
            float2 result[kBatch][kPasses];
            uint32_t hi[kBatch][kPasses], lo[kBatch][kPasses];
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    // (gate_j, up_j, gate_j+1, up_j+1) of the interleaved weight rows; the shadow input makes this a bf16
                    // model, whose SiLU takes the hardware exponential (see silu_fast)
                    const float4 v = value[r][pass];
                    const float a = __fmul_rn(silu_fast(v.x * scale[r]), v.y * scale[r]);
                    const float b = __fmul_rn(silu_fast(v.z * scale[r]), v.w * scale[r]);
                    result[r][pass] = make_float2(a, b);
                    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                    const __nv_bfloat162 l = __floats2bfloat162_rn(a - __low2float(h), b - __high2float(h));
                    hi[r][pass] = *reinterpret_cast<const uint32_t*>(&h);
                    lo[r][pass] = *reinterpret_cast<const uint32_t*>(&l);
                }
            }
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    if (!live[pass]) continue;
                    const int64_t at = static_cast<int64_t>(m0 + rows[r]) * (p.out >> 1) + ((n0 + pass * 128 + lane * 4) >> 1);
                    if (p.y) *reinterpret_cast<float2*>(p.y + at) = result[r][pass];
                    if (p.out_hi) {
                        *reinterpret_cast<uint32_t*>(p.out_hi + at) = hi[r][pass];
                        *reinterpret_cast<uint32_t*>(p.out_lo + at) = lo[r][pass];
                    }
                }
            }
        } else if constexpr (EPI == B200_EPI_STORE) {
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    if (!live[pass]) continue;
                    const float4 v = value[r][pass];
                    const float4 t = make_float4(v.x * scale[r], v.y * scale[r], v.z * scale[r], v.w * scale[r]);
                    const int64_t at = static_cast<int64_t>(m0 + rows[r]) * p.out + n0 + pass * 128 + lane * 4;
                    *reinterpret_cast<float4*>(p.y + at) = t;
                    store_copies(p, at, t);
                }
            }
        } else if constexpr (EPI == B200_EPI_ARGMAX) {
            Candidate best[kBatch];
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
                best[r] = Candidate{-INFINITY, INT32_MAX};
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    const int feature0 = n0 + pass * 128 + lane * 4;
                    const float4 v = value[r][pass];
                    const Candidate low = pair_candidate(feature0, v.x * scale[r], v.y * scale[r], p.out);
                    const Candidate high = pair_candidate(feature0 + 2, v.z * scale[r], v.w * scale[r], p.out);
                    if (live[pass] && preferred(low, best[r])) best[r] = low;
                    if (live[pass] && feature0 + 2 < p.out && preferred(high, best[r])) best[r] = high;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int r = 0; r < kBatch; ++r) {
                    const Candidate other{__shfl_xor_sync(0xffffffffu, best[r].value, o), __shfl_xor_sync(0xffffffffu, best[r].index, o)};
                    if (preferred(other, best[r])) best[r] = other;
                }
            }
            if (lane < kBatch && ready) {
                Candidate mine = best[0];
                int row_of_lane = rows[0];
#pragma unroll
                for (int r = 1; r < kBatch; ++r) {
                    if (lane == r) { mine = best[r]; row_of_lane = rows[r]; }
                }
                p.best_value[static_cast<int64_t>(feature_tile) * p.rows + m0 + row_of_lane] = mine.value;
                p.best_index[static_cast<int64_t>(feature_tile) * p.rows + m0 + row_of_lane] = mine.index;
            }
        } else {
            // q | k | v (src/nn/decoder.cpp:26-28,77-88; src/ops/contraction.cpp:44-49; src/nn/kv_cache.cpp:24-28)
            int2 place[kBatch];
            float2 cosine[kBatch][kPasses], sine[kBatch][kPasses];
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
                place[r] = row_place ? row_place[rows[r]] : qkv_row_place(p, m0 + rows[r]);
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    cosine[r][pass] = make_float2(1.0f, 1.0f);
                    sine[r][pass] = make_float2(0.0f, 0.0f);
                    // (unsigned comparison: the warm-up pass of a caller may see a position that nobody has written yet)
                    const bool turns = region[pass] != 2 && static_cast<unsigned>(place[r].x) < static_cast<unsigned>(p.context)
                                       && n0 + pass * 128 + lane * 4 < p.out;
                    if (turns) {
                        const int64_t at = static_cast<int64_t>(place[r].x) * (p.head_dim >> 1) + (inside[pass] >> 1);
                        cosine[r][pass] = __ldg(reinterpret_cast<const float2*>(p.cosine + at));
                        sine[r][pass] = __ldg(reinterpret_cast<const float2*>(p.sine + at));
                    }
                }
            }
            float4 result[kBatch][kPasses];
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    const float4 v = value[r][pass];
                    result[r][pass] = make_float4(v.x * scale[r], v.y * scale[r], v.z * scale[r], v.w * scale[r]);
                }
            }
            if (p.lora_rank > 0) {
#pragma unroll
                for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                    for (int pass = 0; pass < kPasses; ++pass) {
                        if (region[pass] == 1 || n0 + pass * 128 + lane * 4 >= p.out) continue;
                        float da, db, dc, dd;
                        lora_pair_delta(p, m0 + rows[r], region[pass], local[pass], da, db);
                        lora_pair_delta(p, m0 + rows[r], region[pass], local[pass] + 2, dc, dd);
                        float4& t = result[r][pass];
                        t = make_float4(__fadd_rn(t.x, __fmul_rn(da, p.lora_scale)), __fadd_rn(t.y, __fmul_rn(db, p.lora_scale)),
                                        __fadd_rn(t.z, __fmul_rn(dc, p.lora_scale)), __fadd_rn(t.w, __fmul_rn(dd, p.lora_scale)));
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kBatch; ++r) {
#pragma unroll
                for (int pass = 0; pass < kPasses; ++pass) {
                    // adjacent-pair rotation, each product rounded before the add; v (and positions past the table) keep
                    // cosine 1 and sine 0, which leaves the values as they are
                    const float4 t = result[r][pass];
                    const float2 c = cosine[r][pass], sn = sine[r][pass];
                    float4 turned = t;
                    if (region[pass] != 2) {
                        turned = make_float4(__fsub_rn(__fmul_rn(t.x, c.x), __fmul_rn(t.y, sn.x)), __fadd_rn(__fmul_rn(t.x, sn.x), __fmul_rn(t.y, c.x)),
                                             __fsub_rn(__fmul_rn(t.z, c.y), __fmul_rn(t.w, sn.y)), __fadd_rn(__fmul_rn(t.z, sn.y), __fmul_rn(t.w, c.y)));
                        if (!(static_cast<unsigned>(place[r].x) < static_cast<unsigned>(p.context))) turned = t;
                    }
                    if (!live[pass]) continue;
                    if (region[pass] == 0) {
                        *reinterpret_cast<float4*>(p.q_out + static_cast<int64_t>(m0 + rows[r]) * (p.heads * p.head_dim) + local[pass]) = turned;
                    } else {
                        const int slot = place[r].x % p.kv.page_size;
                        const int64_t at = ((static_cast<int64_t>(place[r].y) * p.kv.kv_heads + head[pass]) * p.kv.page_size + slot) * p.kv.head_dim
                                           + inside[pass];
                        void* pool = p.kv.pool[region[pass] - 1];
                        if (p.kv.dtype == B200_BF16) {
                            const __nv_bfloat162 lo2 = __floats2bfloat162_rn(turned.x, turned.y), hi2 = __floats2bfloat162_rn(turned.z, turned.w);
                            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(pool) + at) =
                                make_uint2(*reinterpret_cast<const uint32_t*>(&lo2), *reinterpret_cast<const uint32_t*>(&hi2));
                        } else {
                            *reinterpret_cast<float4*>(static_cast<float*>(pool) + at) = turned;
                        }
                    }
                }
            }
        }
    }
}

// Finishes the rows [first, last) of a tile held row-major in shared memory (`tile`, or the sum over the cluster's
// `split` partial tiles `peer_tile[z]`).  Warp `worker` of `workers` takes kBatch consecutive rows per iteration: first
// every value the rows need is requested (accumulators from shared memory or from the peers, residual pairs from global
// memory), then the rows are finished, so the memory round trips of the rows overlap instead of queueing behind each
// other.  Lanes run across the feature pairs: every global access is coalesced; per-row reductions are butterflies.
template <int EPI, int kTileN>
__device__ __forceinline__ void finish_rows_pairs(const LinearParams& p, const float* tile, const uint32_t (&peer_tile)[8], int split,
                                            const float* row_scale, int m0, int n0, int feature_tile, int first, int last, int worker,
                                            int workers, int lane, bool ready, const int2* row_place) {
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
                    if (lane == 0 && ready) p.sumsq_out[static_cast<int64_t>(feature_tile) * p.rows + row] = squares;
                }
            }
            if constexpr (EPI == B200_EPI_ARGMAX) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const Candidate other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
                    if (preferred(other, best)) best = other;
                }
                if (lane == 0 && ready) {   // (a caller's warm-up pass hands in accumulators that are not valid: nothing is written)
                    p.best_value[static_cast<int64_t>(feature_tile) * p.rows + row] = best.value;
                    p.best_index[static_cast<int64_t>(feature_tile) * p.rows + row] = best.index;
                }
            }
        }
    }
}

// kForm: 0 = decided here from the call's sizes and addresses, 1 = the caller has checked that the vector form applies
// (rows_take_quads on the host side of its launch), 2 = pairs.  kLocal: the `split` partial tiles all lie in this CTA's own
// shared memory (their senders pushed them here), so they are read with plain shared-memory loads.
template <int EPI, int kTileN, int kForm = 0, bool kLocal = false>
__device__ __forceinline__ void finish_rows(const LinearParams& p, const float* tile, const uint32_t (&peer_tile)[8], int split,
                                            const float* row_scale, int m0, int n0, int feature_tile, int first, int last, int worker,
                                            int workers, int lane, bool ready, const int2* row_place = nullptr) {
    if (kForm == 1 || (kForm == 0 && rows_take_quads<EPI>(p)))
        finish_rows_quads<EPI, kTileN, kLocal>(p, tile, peer_tile, split, row_scale, m0, n0, feature_tile, first, last, worker, workers, lane, ready, row_place);
    else
        finish_rows_pairs<EPI, kTileN>(p, tile, peer_tile, split, row_scale, m0, n0, feature_tile, first, last, worker, workers, lane, ready, row_place);
}

}  // namespace b200
