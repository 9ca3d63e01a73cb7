// K4: masked, scaled row softmax over attention scores.
//
// v[j] = scale * x[j] + (mask[b, j] == 0 ? -10000 : 0);  out = exp(v - max v) / sum
//
// A row lives in the registers of LPR adjacent lanes (LPR = 1..32, a power of two), VPT
// 16-byte vectors per lane, and every lane group works on ROWS rows at once so that
// ROWS * VPT independent 128-bit loads are in flight per thread. Short rows (seq 32 in
// binary16 is 64 bytes) therefore still produce 512-byte contiguous warp accesses. Blocks
// are bound to one batch entry: its columns of the int8 [batch, seq] mask are turned into
// additive float terms once (in registers for short rows, in shared memory for long ones) and
// reused for every row of that entry; the reference's score-sized broadcast mask tensor never exists. Arithmetic is
// float32 issued as packed .f32x2. HBM traffic: one read and one write of the score matrix.
#include "common.cuh"

namespace cubk {

constexpr float kMaskedScore = -10000.0f;  // src/cuBERT/op_att/AttentionSelf.cpp:58-60
constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ void load_mask_add(const int8_t *mask_row, int idx, float (&add)[Vec<T>::EPV]);

template <>
__device__ __forceinline__ void load_mask_add<float>(const int8_t *mask_row, int idx, float (&add)[4]) {
    const uint32_t m = __ldg(reinterpret_cast<const uint32_t *>(mask_row) + idx);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        add[e] = ((m >> (8 * e)) & 0xffu) == 0 ? kMaskedScore : 0.f;
    }
}

template <>
__device__ __forceinline__ void load_mask_add<__half>(const int8_t *mask_row, int idx, float (&add)[8]) {
    const uint2 m = __ldg(reinterpret_cast<const uint2 *>(mask_row) + idx);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        add[e] = ((m.x >> (8 * e)) & 0xffu) == 0 ? kMaskedScore : 0.f;
        add[4 + e] = ((m.y >> (8 * e)) & 0xffu) == 0 ? kMaskedScore : 0.f;
    }
}

// Work is cut into items of ROWS_PER_BLOCK consecutive rows of one batch entry (all of whose
// rows share one mask row). Every block takes a contiguous range of items, so it changes batch
// entry rarely; when it does, each thread converts its columns of the mask into additive terms,
// which then stay in registers for all the rows that follow.
// MASK_SMEM: the additive terms live in shared memory (float32, [EPV/4][nvec] so that 128-bit reads
// are conflict-free) instead of in registers; long rows then need half the registers, and twice as
// many warps stay resident.
// EXTENTS: key_extents[b] = n says that every key of batch entry b from column n on is masked out (and
// at least one below n is kept). Vectors that lie entirely at or beyond n are then not read at all:
// their probabilities are exactly 0, which is what the full computation gives them. They are written
// as zeros up to column max(n, zero_to) and left untouched beyond it (a consumer that reads only the
// first n columns of this entry needs no zeros after them).
template <typename T, int LPR, int VPT, int ROWS, int BLOCK, bool MASK_SMEM, bool EXTENTS>
__global__ void __launch_bounds__(BLOCK)
masked_softmax_kernel(const T *scores, const int8_t *mask, T *out, uint32_t rows_per_batch, int seq, int nvec,
                      float scale, uint32_t total_items, FastDiv items_per_batch, const int32_t *key_extents,
                      int zero_to) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    extern __shared__ float4 s_madd[];
    constexpr int GPW = 32 / LPR;                          // row groups per warp
    constexpr int ROWS_PER_BLOCK = (BLOCK / 32) * GPW * ROWS;  // rows of one item
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR;
    const int l = lane % LPR;
    const int warp = threadIdx.x >> 5;

    // items split as evenly as possible: the first `extra` blocks take one more
    const uint32_t share = total_items / gridDim.x;
    const uint32_t extra = total_items - share * gridDim.x;
    const uint32_t item_begin = blockIdx.x * share + min(blockIdx.x, extra);
    const uint32_t item_end = item_begin + share + (blockIdx.x < extra ? 1u : 0u);

    float2 madd[MASK_SMEM ? 1 : VPT][PAIRS];
#pragma unroll
    for (int k = 0; k < (MASK_SMEM ? 1 : VPT); ++k) {
#pragma unroll
        for (int e = 0; e < PAIRS; ++e) {
            madd[k][e] = make_float2(0.f, 0.f);
        }
    }
    uint32_t cur_b = 0xffffffffu;
    const float2 scale2 = splat2(scale);
    const float2 log2e2 = splat2(kLog2e);
    // per vector of this lane: read and reduced (in_use), written (stored); all true without extents
    bool in_use[VPT], stored[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        in_use[k] = stored[k] = l + k * LPR < nvec;
    }

    for (uint32_t item = item_begin; item < item_end; ++item) {
        const uint32_t b = fast_div(item, items_per_batch);
        if (EXTENTS && b != cur_b) {
            const int n = min(max(__ldg(key_extents + b), 1), seq);
            const int write_to = max(n, zero_to);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int first_col = (l + k * LPR) * EPV;
                in_use[k] = first_col < n;
                stored[k] = first_col < min(write_to, seq);
            }
        }
        if (b != cur_b && MASK_SMEM) {  // uniform over the block: all its threads walk the same items
            cur_b = b;
            __syncthreads();  // the previous entry's terms are no longer read
            for (int idx = threadIdx.x; idx < nvec; idx += BLOCK) {
                float add[EPV];
                if (mask != nullptr) {
                    load_mask_add<T>(mask + (size_t) b * seq, idx, add);
                } else {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        add[e] = 0.f;
                    }
                }
#pragma unroll
                for (int q = 0; q < EPV / 4; ++q) {
                    s_madd[q * nvec + idx] = make_float4(add[4 * q], add[4 * q + 1], add[4 * q + 2], add[4 * q + 3]);
                }
            }
            __syncthreads();
        }
        if (b != cur_b) {
            cur_b = b;
            if (mask != nullptr) {
#pragma unroll
                for (int k = 0; k < (MASK_SMEM ? 0 : VPT); ++k) {
                    const int idx = l + k * LPR;
                    if (idx < nvec) {
                        float add[EPV];
                        load_mask_add<T>(mask + (size_t) b * seq, idx, add);
#pragma unroll
                        for (int e = 0; e < PAIRS; ++e) {
                            madd[k][e] = make_float2(add[2 * e], add[2 * e + 1]);
                        }
                    }
                }
            }
        }
        const uint64_t batch_row0 = (uint64_t) b * rows_per_batch;
        const uint32_t r0 = (item - b * items_per_batch.div) * ROWS_PER_BLOCK + warp * (GPW * ROWS);
        if (r0 >= rows_per_batch) {
            continue;  // the whole warp skips together
        }
        uint4 raw[ROWS][VPT];
        bool live[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const uint32_t rb = r0 + r * GPW + sub;
            live[r] = rb < rows_per_batch;
            const T *src = scores + (batch_row0 + rb) * (uint64_t) seq;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int idx = l + k * LPR;
                raw[r][k] = (live[r] && in_use[k]) ? ld_stream(src + (size_t) idx * EPV) : make_uint4(0, 0, 0, 0);
            }
        }

#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float2 v[VPT][PAIRS];
            float mx = -3.0e38f;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                Vec2<T>::unpack(raw[r][k], v[k]);
                if (in_use[k]) {
                    float2 m[PAIRS];
                    if (MASK_SMEM) {
#pragma unroll
                        for (int q = 0; q < EPV / 4; ++q) {
                            const float4 f = s_madd[q * nvec + l + k * LPR];
                            m[2 * q] = make_float2(f.x, f.y);
                            m[2 * q + 1] = make_float2(f.z, f.w);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < PAIRS; ++e) {
                        v[k][e] = fma2(scale2, v[k][e], MASK_SMEM ? m[e] : madd[MASK_SMEM ? 0 : k][e]);
                        mx = fmaxf(mx, fmaxf(v[k][e].x, v[k][e].y));
                    }
                }
            }
            mx = group_max<LPR>(mx);

            // exp(v - mx) = 2^(v * log2e - mx * log2e): the product is exact inside the FMA and the
            // rounding of mx * log2e is a factor common to the whole row, which the division removes.
            const float2 neg_mx = splat2(-mx * kLog2e);
            float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                if (in_use[k]) {
#pragma unroll
                    for (int e = 0; e < PAIRS; ++e) {
                        const float2 t = fma2(v[k][e], log2e2, neg_mx);
                        v[k][e] = make_float2(fast_exp2(t.x), fast_exp2(t.y));
                        sum2 = add2(sum2, v[k][e]);
                    }
                }
            }
            const float sum = group_sum<LPR>(sum2.x + sum2.y);
            const float2 inv = splat2(1.f / sum);

            if (live[r]) {
                T *dst = out + (batch_row0 + r0 + r * GPW + sub) * (uint64_t) seq;
#pragma unroll
                for (int k = 0; k < VPT; ++k) {
                    const int idx = l + k * LPR;
                    if (in_use[k]) {
#pragma unroll
                        for (int e = 0; e < PAIRS; ++e) {
                            v[k][e] = mul2(v[k][e], inv);
                        }
                        st_vec(dst + (size_t) idx * EPV, Vec2<T>::pack(v[k]));
                    } else if (EXTENTS && stored[k]) {
                        st_vec(dst + (size_t) idx * EPV, make_uint4(0, 0, 0, 0));
                    }
                }
            }
        }
    }
}

// Any row length, any alignment: one warp per row, three scalar passes. Key extents as above, by column.
template <typename T>
__global__ void __launch_bounds__(128)
masked_softmax_generic_kernel(const T *scores, const int8_t *mask, T *out, int64_t rows, int64_t rows_per_batch,
                              int seq, float scale, const int32_t *key_extents, int zero_to) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t) blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) {
        return;
    }
    const T *src = scores + row * seq;
    T *dst = out + row * seq;
    const int64_t b = row / rows_per_batch;
    const int8_t *mask_row = mask != nullptr ? mask + b * seq : nullptr;
    const int n = key_extents != nullptr ? min(max(key_extents[b], 1), seq) : seq;
    const int write_to = key_extents != nullptr ? min(max(n, zero_to), seq) : seq;
    float mx = -3.0e38f;
    for (int j = lane; j < n; j += 32) {
        const float add = (mask_row != nullptr && mask_row[j] == 0) ? kMaskedScore : 0.f;
        mx = fmaxf(mx, fmaf(scale, to_float<T>(src[j]), add));
    }
    mx = group_max<32>(mx);
    float sum = 0.f;
    for (int j = lane; j < n; j += 32) {
        const float add = (mask_row != nullptr && mask_row[j] == 0) ? kMaskedScore : 0.f;
        sum += fast_exp2((fmaf(scale, to_float<T>(src[j]), add) - mx) * kLog2e);
    }
    sum = group_sum<32>(sum);
    const float inv = 1.f / sum;
    for (int j = lane; j < write_to; j += 32) {
        float p = 0.f;
        if (j < n) {
            const float add = (mask_row != nullptr && mask_row[j] == 0) ? kMaskedScore : 0.f;
            p = fast_exp2((fmaf(scale, to_float<T>(src[j]), add) - mx) * kLog2e) * inv;
        }
        dst[j] = from_float<T>(p);
    }
}

// Rows of four or more vectors per lane keep the additive mask terms in shared memory by default.
// Inside a BERT step, where the GEMMs hold the GPU at its power cap (SM clock 1.3-1.6 GHz), the lower
// register count wins: BERT-large seq 512 binary16 1621 -> 1496 us per launch, BERT-base seq 128
// 34.1 -> 32.7 us. Timed alone at 1.9 GHz the register variant is ahead (1353 against 1410 us on the
// same 8.6 GB). CUBK_OPT_SOFTMAX_MASK_SMEM = 0 selects the register variant.
static bool mask_in_smem() {
    return option(CUBK_OPT_SOFTMAX_MASK_SMEM) != 0;
}

template <typename T>
int masked_softmax(const T *scores, const int8_t *mask, int64_t rows, int64_t rows_per_batch, int seq,
                   float scale, T *out, cudaStream_t stream, const int32_t *key_extents = nullptr,
                   int zero_to = 0) {
    if (scores == nullptr || out == nullptr || rows < 0 || seq <= 0 || (mask != nullptr && rows_per_batch <= 0) ||
        (key_extents != nullptr && (mask == nullptr || zero_to < 0))) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (rows == 0) {
        return CUBK_OK;
    }
    if (rows > 0x7fffffffLL) {
        return CUBK_ERR_UNSUPPORTED;
    }
    if (mask == nullptr) {
        rows_per_batch = rows;
    }
    constexpr int EPV = Vec<T>::EPV;
    constexpr int BLOCK = 256;
    const int nvec = seq / EPV;
    const int64_t batches = rows / rows_per_batch;
    const bool vec_ok = seq % EPV == 0 && nvec <= 256 && aligned16(scores) && aligned16(out) &&
                        (mask == nullptr || aligned8(mask)) && rows_per_batch <= 0x7fffffffLL &&
                        rows % rows_per_batch == 0;
    if (vec_ok) {
#define LAUNCH_AS(LPR, VPT, ROWS, MASK_SMEM)                                                            \
    if (key_extents != nullptr) LAUNCH_WITH(LPR, VPT, ROWS, MASK_SMEM, true) else LAUNCH_WITH(LPR, VPT, ROWS, MASK_SMEM, false)
#define LAUNCH_WITH(LPR, VPT, ROWS, MASK_SMEM, EXTENTS)                                                 \
    {                                                                                                   \
        static OccupancyCache cache;                                                                    \
        auto kernel = masked_softmax_kernel<T, LPR, VPT, ROWS, BLOCK, MASK_SMEM, EXTENTS>;              \
        const size_t smem = MASK_SMEM ? sizeof(float) * (size_t) seq : 0;                               \
        const int64_t rows_per_block = (int64_t) (BLOCK / 32) * (32 / LPR) * ROWS;                      \
        const int64_t per_batch = (rows_per_batch + rows_per_block - 1) / rows_per_block;               \
        const int64_t items = per_batch * batches;                                                      \
        int64_t grid = resident_blocks(kernel, BLOCK, smem, &cache);                                    \
        if (grid > items) grid = items;                                                                 \
        kernel<<<(unsigned) grid, BLOCK, smem, stream>>>(scores, mask, out, (uint32_t) rows_per_batch,  \
                                                         seq, nvec, scale, (uint32_t) items,            \
                                                         make_fastdiv((uint32_t) per_batch), key_extents,\
                                                         zero_to);                                      \
    }
#define LAUNCH(LPR, VPT, ROWS) LAUNCH_AS(LPR, VPT, ROWS, false)
#define LAUNCH_LONG(LPR, VPT, ROWS)                                  \
    if (mask_in_smem()) LAUNCH_AS(LPR, VPT, ROWS, true) else LAUNCH_AS(LPR, VPT, ROWS, false)
        if (nvec <= 1) {
            LAUNCH(1, 1, 4);
        } else if (nvec <= 2) {
            LAUNCH(2, 1, 4);
        } else if (nvec <= 4) {
            LAUNCH(4, 1, 4);
        } else if (nvec <= 8) {
            LAUNCH(8, 1, 4);
        } else if (nvec <= 16) {
            // fewer lanes per row: 2 shuffle steps per reduction instead of 4
            LAUNCH_LONG(4, 4, 1)
        } else if (nvec <= 32) {
            LAUNCH(32, 1, 4);
        } else if (nvec <= 64) {
            LAUNCH_LONG(16, 4, 1)
        } else if (nvec <= 128) {
            LAUNCH_LONG(32, 4, 1)
        } else {
            LAUNCH_LONG(32, 8, 1)
        }
#undef LAUNCH_LONG
#undef LAUNCH
#undef LAUNCH_AS
#undef LAUNCH_WITH
    } else {
        const int64_t grid = (rows + 3) / 4;
        masked_softmax_generic_kernel<T><<<(unsigned) grid, 128, 0, stream>>>(scores, mask, out, rows,
                                                                             rows_per_batch, seq, scale,
                                                                             key_extents, zero_to);
    }
    return check_launch();
}

}  // namespace cubk

extern "C" {

int cubk_masked_softmax_f32(const float *scores, const int8_t *mask, int64_t rows, int64_t rows_per_batch,
                            int seq, float scale, float *out, void *stream) {
    return cubk::masked_softmax<float>(scores, mask, rows, rows_per_batch, seq, scale, out,
                                       (cudaStream_t) stream);
}

int cubk_masked_softmax_f16(const void *scores, const int8_t *mask, int64_t rows, int64_t rows_per_batch,
                            int seq, float scale, void *out, void *stream) {
    return cubk::masked_softmax<__half>((const __half *) scores, mask, rows, rows_per_batch, seq, scale,
                                        (__half *) out, (cudaStream_t) stream);
}

int cubk_masked_softmax_extents_f32(const float *scores, const int8_t *mask, const int32_t *key_extents, int zero_to,
                                    int64_t rows, int64_t rows_per_batch, int seq, float scale, float *out,
                                    void *stream) {
    if (key_extents == nullptr) {
        return CUBK_ERR_INVALID_ARG;
    }
    return cubk::masked_softmax<float>(scores, mask, rows, rows_per_batch, seq, scale, out, (cudaStream_t) stream,
                                       key_extents, zero_to);
}

int cubk_masked_softmax_extents_f16(const void *scores, const int8_t *mask, const int32_t *key_extents, int zero_to,
                                    int64_t rows, int64_t rows_per_batch, int seq, float scale, void *out,
                                    void *stream) {
    if (key_extents == nullptr) {
        return CUBK_ERR_INVALID_ARG;
    }
    return cubk::masked_softmax<__half>((const __half *) scores, mask, rows, rows_per_batch, seq, scale,
                                        (__half *) out, (cudaStream_t) stream, key_extents, zero_to);
}

}
