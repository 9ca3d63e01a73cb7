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

// ------------------------------------------------------------------ whole attention of short sequences
// For requests of a few hundred tokens the forward pass is bound by its chain of dependent launches, not
// by work: the scores of one (sequence, head) are a 32 x 32 or 64 x 64 tile. This kernel does Q.K^T, the
// masked softmax and P.V of one (sequence, head) per block on the ordinary float32 pipes, in place of two
// batched library products and K4: two launches fewer per layer. It rounds where the three-launch path
// rounds (scores and probabilities pass through the storage type), so the results differ from that
// path only by the order of the additions inside the two dot products.
//   qkv      [batch * seq, 3 * hidden]: per token Q | K | V, head h at columns h * 64 of each part
//   context  [batch * seq, hidden]
constexpr int kSmallHeadDim = 64;
constexpr int kSmallAttentionWarps = 8;   // query rows per block: one per warp
constexpr int kSmallKeyStride = kSmallHeadDim + 4;   // floats per K row in shared memory: 128-bit reads by 32
                                                     // lanes of 32 different rows are conflict-free at 68

// Block = (sequence, head) x a group of 8 query rows. K and V of the head go to shared memory as float32
// (every block of the head's groups loads them again: 16 KB from L2), then each warp takes one query row:
// lane j owns key j (and j + 32 when seq > 32) for the scores and the softmax, columns 2 * lane and
// 2 * lane + 1 for the context.
template <typename T, int SMAX, int RPW>
__global__ void __launch_bounds__(32 * kSmallAttentionWarps, (SMAX == 64 && RPW == 2 ? 2 : 1))
small_attention_kernel(const T *qkv, const int8_t *mask, T *context, int seq, int heads, int hidden, float scale) {
    constexpr int D = kSmallHeadDim;
    constexpr int KPL = SMAX / 32;  // keys per lane
    constexpr int ROWS = kSmallAttentionWarps * RPW;   // query rows per block, RPW of them per warp
    __shared__ __align__(16) float s_k[SMAX][kSmallKeyStride];
    __shared__ __align__(16) float s_v[SMAX][D];
    __shared__ __align__(16) float s_q[ROWS][D];
    __shared__ __align__(16) float s_p[ROWS][SMAX];
    __shared__ float s_madd[SMAX];
    const int b = blockIdx.x / heads;
    const int h = blockIdx.x - b * heads;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const size_t row_stride = 3 * (size_t) hidden;
    const T *base = qkv + (size_t) b * seq * row_stride + (size_t) h * D;

    // K and V: pairs of adjacent columns per thread (4- or 8-byte loads, a row of 64 columns per warp)
    for (int i = threadIdx.x; i < seq * (D / 2); i += blockDim.x) {
        const int j = i / (D / 2), c = 2 * (i - j * (D / 2));
        const T *kp = base + (size_t) j * row_stride + hidden + c;
        const T *vp = kp + hidden;
        s_k[j][c] = to_float<T>(kp[0]);
        s_k[j][c + 1] = to_float<T>(kp[1]);
        s_v[j][c] = to_float<T>(vp[0]);
        s_v[j][c + 1] = to_float<T>(vp[1]);
    }
    for (int j = threadIdx.x; j < SMAX; j += blockDim.x) {
        s_madd[j] = (j < seq && (mask == nullptr || mask[(size_t) b * seq + j] != 0)) ? 0.f : kMaskedScore;
    }
    const int row0 = blockIdx.y * ROWS + warp * RPW;   // this warp's first query row
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        if (row0 + r < seq) {
            const T *qp = base + (size_t) (row0 + r) * row_stride + 2 * lane;
            s_q[warp * RPW + r][2 * lane] = to_float<T>(qp[0]);
            s_q[warp * RPW + r][2 * lane + 1] = to_float<T>(qp[1]);
        }
    }
    __syncthreads();
    if (row0 >= seq) {
        return;
    }

    // scores of RPW rows at once (independent chains), softmax per row
    float v[RPW][KPL];
    float mx[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        mx[r] = -3.0e38f;
    }
#pragma unroll
    for (int u = 0; u < KPL; ++u) {
        const int j = lane + 32 * u;
        const int jr = j < seq ? j : 0;   // rows past the sequence are not staged: read row 0, discard
        float4 acc[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int c = 0; c < D; c += 4) {
            const float4 k4 = *reinterpret_cast<const float4 *>(&s_k[jr][c]);
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const float4 q4 = *reinterpret_cast<const float4 *>(&s_q[warp * RPW + r][c]);
                acc[r].x = fmaf(q4.x, k4.x, acc[r].x);
                acc[r].y = fmaf(q4.y, k4.y, acc[r].y);
                acc[r].z = fmaf(q4.z, k4.z, acc[r].z);
                acc[r].w = fmaf(q4.w, k4.w, acc[r].w);
            }
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const float dot = (acc[r].x + acc[r].y) + (acc[r].z + acc[r].w);
            // the stored score (storage precision), then the additive mask, as K4 reads it
            v[r][u] = j < seq ? to_float<T>(from_float<T>(scale * dot)) + s_madd[j] : -3.0e38f;
            mx[r] = fmaxf(mx[r], v[r][u]);
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const float m = group_max<32>(mx[r]);
        float p[KPL];
        float sum = 0.f;
#pragma unroll
        for (int u = 0; u < KPL; ++u) {
            p[u] = lane + 32 * u < seq ? fast_exp2(fmaf(v[r][u], kLog2e, -m * kLog2e)) : 0.f;
            sum += p[u];
        }
        sum = group_sum<32>(sum);
        const float inv = 1.f / sum;
#pragma unroll
        for (int u = 0; u < KPL; ++u) {
            s_p[warp * RPW + r][lane + 32 * u] = to_float<T>(from_float<T>(p[u] * inv));  // the stored probability
        }
    }
    __syncwarp();
    // context columns 2 * lane and 2 * lane + 1 of the RPW rows; keys past the sequence are never read
    float2 acc[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        acc[r] = make_float2(0.f, 0.f);
    }
    for (int j = 0; j < seq; ++j) {
        const float2 vv = *reinterpret_cast<const float2 *>(&s_v[j][2 * lane]);
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const float pj = s_p[warp * RPW + r][j];
            acc[r].x = fmaf(pj, vv.x, acc[r].x);
            acc[r].y = fmaf(pj, vv.y, acc[r].y);
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        if (row0 + r < seq) {
            T *dst = context + ((size_t) b * seq + row0 + r) * hidden + (size_t) h * D + 2 * lane;
            if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(dst) & 3u) == 0) {
                *reinterpret_cast<__half2 *>(dst) = __floats2half2_rn(acc[r].x, acc[r].y);
            } else {
                dst[0] = from_float<T>(acc[r].x);
                dst[1] = from_float<T>(acc[r].y);
            }
        }
    }
}

// ---- binary16 storage, up to 128 positions: the same computation on warp-level matrix instructions
// The scores of one (sequence, head) never leave the SM: a warp keeps a strip of 16 query rows in registers
// from Q.K^T (mma.sync m16n8k16, binary16 in, float32 accumulators: what the library's products of binary16
// matrices accumulate in as well) through the masked softmax to P.V, rounding scores and probabilities to
// binary16 where the three-launch path stores them. Against that path a layer of 256 x 128 tokens no longer
// writes and re-reads its 100 MB score matrix three times; against the float32-pipe kernel above the
// shared-memory traffic falls by ten (ldmatrix moves 512 B per instruction). A 32 x 32 x 64 or 128 x 128 x 64
// product per head is below what a tcgen05 tile (operands through shared-memory descriptors, accumulators in
// tensor memory behind an mbarrier, 64 or 128 rows per instruction) is made for: with the softmax between the
// two products the accumulators have to come back to registers anyway, and the kernel is bound by the
// latency of a launch (short requests) or by reading Q | K | V once from HBM (long ones), not by arithmetic.
//
// Block = one (sequence, head); warp w owns query rows 16 w .. 16 w + 15 and loads them straight into
// A-operand registers. K and V of the head are staged as binary16 rows of 64 + 8 elements (144 B: the eight
// 16-byte rows of an 8 x 8 ldmatrix tile fall into eight different bank groups); rows at and beyond seq are
// zero so that a probability of 0 never meets a stray NaN. Fragment layouts are those of the PTX ISA for
// mma.m16n8k16: with g = lane / 4, t = lane % 4 a thread holds accumulator elements (g, 2t), (g, 2t+1),
// (g+8, 2t), (g+8, 2t+1) of every 16 x 8 tile, which is also how the A operand of the second product wants
// the probabilities.
constexpr int kMmaRowHalves = kSmallHeadDim + 8;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_row) {
    const uint32_t a = (uint32_t) __cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row) {
    const uint32_t a = (uint32_t) __cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}

// d += a (16 x 16, row-major) . b (16 x 8, column-major), binary16 operands, float32 accumulators;
// d[0] = elements (g, 2t), (g, 2t+1), d[1] = elements (g+8, 2t), (g+8, 2t+1)
__device__ __forceinline__ void mma_16x8x16(float2 (&d)[2], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0].x), "+f"(d[0].y), "+f"(d[1].x), "+f"(d[1].y)
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int SMAX, int STRIPS>
__global__ void __launch_bounds__(2 * SMAX / STRIPS, SMAX == 128 ? 4 : 1)
small_attention_mma_kernel(const __half *qkv, const int8_t *mask, __half *context, int seq, int heads, int hidden,
                           float scale) {
    constexpr int D = kSmallHeadDim;
    constexpr int LD = kMmaRowHalves;
    constexpr int WARPS = SMAX / 16 / STRIPS;   // each warp takes STRIPS strips of 16 query rows, one after the other
    constexpr int THREADS = 32 * WARPS;
    constexpr int VPT = SMAX * 8 / THREADS;     // 16-byte vectors of K (and of V) staged per thread
    constexpr int NT = SMAX / 8;                // 8-key tiles of a score strip
    constexpr int KS = SMAX / 16;               // 16-key steps of the second product
    static_assert(THREADS >= SMAX || SMAX <= 64, "the key extent is found with one key per thread");
    __shared__ __align__(16) __half s_k[SMAX][LD];
    __shared__ __align__(16) __half s_v[SMAX][LD];
    __shared__ __align__(8) float s_madd[SMAX];
    __shared__ int s_last[SMAX / 32];
    const int b = blockIdx.x / heads;
    const int h = blockIdx.x - b * heads;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const size_t row_stride = 3 * (size_t) hidden;
    const __half *base = qkv + (size_t) b * seq * row_stride + (size_t) h * D;

    // the Q rows of this warp's strips go straight into A-operand registers (rows g and g + 8, four
    // 16-column steps); rows at and beyond seq are zeros and their results are dropped
    uint32_t qa[STRIPS][D / 16][4];
#pragma unroll
    for (int s = 0; s < STRIPS; ++s) {
        const int m0 = 16 * (warp + WARPS * s);
        const bool live0 = m0 + g < seq, live1 = m0 + g + 8 < seq;
        const __half *q0 = base + (size_t) (m0 + g) * row_stride + 2 * t;
        const __half *q1 = q0 + 8 * row_stride;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            qa[s][kk][0] = live0 ? __ldg(reinterpret_cast<const uint32_t *>(q0 + 16 * kk)) : 0u;
            qa[s][kk][1] = live1 ? __ldg(reinterpret_cast<const uint32_t *>(q1 + 16 * kk)) : 0u;
            qa[s][kk][2] = live0 ? __ldg(reinterpret_cast<const uint32_t *>(q0 + 16 * kk + 8)) : 0u;
            qa[s][kk][3] = live1 ? __ldg(reinterpret_cast<const uint32_t *>(q1 + 16 * kk + 8)) : 0u;
        }
    }
    // additive mask terms; for long sequences also the key extent of this sequence: one past its last kept key.
    // Keys from there on are all masked: their probabilities are exactly 0 (exp of about -10000 below the
    // row's largest score), so they are neither loaded nor multiplied. No kept key at all: every key counts.
    int ext = seq;
    for (int j = threadIdx.x; j < SMAX; j += THREADS) {   // whole warps
        const bool kept = j < seq && (mask == nullptr || mask[(size_t) b * seq + j] != 0);
        s_madd[j] = kept ? 0.f : kMaskedScore;
        if constexpr (SMAX > 64) {
            const unsigned ballot = __ballot_sync(0xffffffffu, kept);
            if (lane == 0) {
                s_last[j >> 5] = ballot != 0u ? (j & ~31) + 32 - __clz(ballot) : 0;
            }
        }
    }
    if constexpr (SMAX > 64) {
        __syncthreads();
        int last = 0;
#pragma unroll
        for (int w = 0; w < SMAX / 32; ++w) {
            last = max(last, s_last[w]);
        }
        ext = last > 0 ? last : seq;
    }
    const int ext16 = (ext + 15) & ~15;   // the key rows the products touch (at most SMAX)
    // stage K | V: eight 16-byte vectors per row, all loads issued before the first store; rows in
    // [ext, ext16) are zeros, rows beyond are never read
    {
        uint4 k[VPT], v[VPT];
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const int i = threadIdx.x + u * THREADS;
            const int j = i >> 3, c = (i & 7) * 8;
            if (j < ext) {
                const __half *p = base + (size_t) j * row_stride + hidden + c;
                k[u] = __ldg(reinterpret_cast<const uint4 *>(p));
                v[u] = __ldg(reinterpret_cast<const uint4 *>(p + hidden));
            } else {
                k[u] = v[u] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const int i = threadIdx.x + u * THREADS;
            const int j = i >> 3, c = (i & 7) * 8;
            if (j < ext16) {
                *reinterpret_cast<uint4 *>(&s_k[j][c]) = k[u];
                *reinterpret_cast<uint4 *>(&s_v[j][c]) = v[u];
            }
        }
    }
    __syncthreads();

    const float2 scale2 = splat2(scale);
    const float2 log2e2 = splat2(kLog2e);
    constexpr float kLeftOut = -1.0e30f;   // a column at or beyond the extent: exp2 gives it exactly 0
#pragma unroll
    for (int s = 0; s < STRIPS; ++s) {
        const int m0 = 16 * (warp + WARPS * s);
        if (m0 >= seq) {
            break;   // the strips of a warp ascend
        }
        // scores of the strip: S[16, SMAX] = Q[16, 64] . K^T; sc[n][0] = row g, sc[n][1] = row g + 8 of tile n
        float2 sc[NT][2];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            sc[n][0] = sc[n][1] = make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int n = 0; n < NT; n += 2) {
                if (8 * n >= ext16) {
                    break;   // uniform over the block
                }
                uint32_t kb[4];
                // tiles: keys 8n..8n+7 at columns 16 kk and 16 kk + 8, then keys 8n+8..8n+15 likewise
                ldmatrix_x4(kb, &s_k[8 * n + (lane & 7) + 8 * (lane >> 4)][16 * kk + 8 * ((lane >> 3) & 1)]);
                mma_16x8x16(sc[n], qa[s][kk], kb[0], kb[1]);
                mma_16x8x16(sc[n + 1], qa[s][kk], kb[2], kb[3]);
            }
        }

        // masked softmax of rows g and g + 8; a row lives in the four lanes of a quad. The stored score
        // (storage precision), then the additive mask, as K4 reads it.
        float mx0 = -3.0e38f, mx1 = -3.0e38f;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if (8 * n >= ext16) {
                break;
            }
            const int col = 8 * n + 2 * t;
            const float2 madd = *reinterpret_cast<const float2 *>(&s_madd[col]);
            float2 r0 = __half22float2(__float22half2_rn(mul2(sc[n][0], scale2)));
            float2 r1 = __half22float2(__float22half2_rn(mul2(sc[n][1], scale2)));
            r0 = add2(r0, madd);
            r1 = add2(r1, madd);
            if (col >= ext) {
                r0.x = r1.x = kLeftOut;
            }
            if (col + 1 >= ext) {
                r0.y = r1.y = kLeftOut;
            }
            sc[n][0] = r0;
            sc[n][1] = r1;
            mx0 = fmaxf(mx0, fmaxf(r0.x, r0.y));
            mx1 = fmaxf(mx1, fmaxf(r1.x, r1.y));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float2 nm0 = splat2(-mx0 * kLog2e), nm1 = splat2(-mx1 * kLog2e);
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if (8 * n >= ext16) {
                break;
            }
            float2 e0 = fma2(sc[n][0], log2e2, nm0), e1 = fma2(sc[n][1], log2e2, nm1);
            e0 = make_float2(fast_exp2(e0.x), fast_exp2(e0.y));
            e1 = make_float2(fast_exp2(e1.x), fast_exp2(e1.y));
            acc0 = add2(acc0, e0);
            acc1 = add2(acc1, e1);
            sc[n][0] = e0;
            sc[n][1] = e1;
        }
        float sum0 = acc0.x + acc0.y, sum1 = acc1.x + acc1.y;
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        const float2 inv0 = splat2(1.f / sum0), inv1 = splat2(1.f / sum1);
        // the stored probabilities, packed as the A operand of the second product
        uint32_t pr[NT][2];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const __half2 p0 = __float22half2_rn(mul2(sc[n][0], inv0));
            const __half2 p1 = __float22half2_rn(mul2(sc[n][1], inv1));
            pr[n][0] = *reinterpret_cast<const uint32_t *>(&p0);
            pr[n][1] = *reinterpret_cast<const uint32_t *>(&p1);
        }

        // context of the strip: O[16, 64] = P[16, SMAX] . V[SMAX, 64]
        float2 o[D / 8][2];
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            o[n][0] = o[n][1] = make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            if (16 * kk >= ext16) {
                break;
            }
            const uint32_t a[4] = {pr[2 * kk][0], pr[2 * kk][1], pr[2 * kk + 1][0], pr[2 * kk + 1][1]};
#pragma unroll
            for (int n = 0; n < D / 8; n += 2) {
                uint32_t vb[4];
                // transposed tiles: keys 16 kk..+7 and 16 kk + 8..+15 at columns 8n, then the same keys at 8n + 8
                ldmatrix_x4_trans(vb, &s_v[16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1)][8 * n + 8 * (lane >> 4)]);
                mma_16x8x16(o[n], a, vb[0], vb[1]);
                mma_16x8x16(o[n + 1], a, vb[2], vb[3]);
            }
        }
        __half *out0 = context + ((size_t) b * seq + m0 + g) * hidden + (size_t) h * D + 2 * t;
        __half *out1 = out0 + 8 * (size_t) hidden;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            if (m0 + g < seq) {
                *reinterpret_cast<__half2 *>(out0 + 8 * n) = __float22half2_rn(o[n][0]);
            }
            if (m0 + g + 8 < seq) {
                *reinterpret_cast<__half2 *>(out1 + 8 * n) = __float22half2_rn(o[n][1]);
            }
        }
    }
}

template <typename T>
constexpr int kSmallAttentionMaxSeq = sizeof(T) == 2 ? 128 : 64;

template <typename T>
int small_attention(const T *qkv, const int8_t *mask, int batch, int seq, int heads, int hidden, float scale, T *context,
                    cudaStream_t stream) {
    if (qkv == nullptr || context == nullptr || batch < 0 || seq <= 0 || heads <= 0 || hidden <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (seq > kSmallAttentionMaxSeq<T> || hidden != heads * kSmallHeadDim || (int64_t) batch * heads > 0x7fffffffLL) {
        return CUBK_ERR_UNSUPPORTED;
    }
    if (batch == 0) {
        return CUBK_OK;
    }
    if constexpr (sizeof(T) == 2) {
        // 16-byte vectors of K | V rows (their strides are multiples of 128 bytes), 4-byte loads and stores
        if ((reinterpret_cast<uintptr_t>(qkv) & 15u) == 0 && (reinterpret_cast<uintptr_t>(context) & 3u) == 0) {
            const unsigned blocks = (unsigned) (batch * heads);
            if (seq <= 32) {
                small_attention_mma_kernel<32, 1><<<blocks, 64, 0, stream>>>(qkv, mask, context, seq, heads, hidden, scale);
            } else if (seq <= 64) {
                small_attention_mma_kernel<64, 1><<<blocks, 128, 0, stream>>>(qkv, mask, context, seq, heads, hidden, scale);
            } else {
                small_attention_mma_kernel<128, 2><<<blocks, 128, 0, stream>>>(qkv, mask, context, seq, heads, hidden, scale);
            }
            return check_launch();
        }
        if (seq > 64) {
            return CUBK_ERR_UNSUPPORTED;  // the float32-pipe kernel below stops at 64 positions
        }
    }
    // one query row per warp while that already gives every SM a few blocks, two rows per warp beyond
    // (half the blocks, each loading K and V once for twice the rows)
    const bool two_rows = (int64_t) batch * heads * ((seq + 7) / 8) > 2 * 148;
    const int rows = kSmallAttentionWarps * (two_rows ? 2 : 1);
    const dim3 grid((unsigned) (batch * heads), (unsigned) ((seq + rows - 1) / rows));
#define SMALL_ATTENTION(SMAX, RPW)                                                                              \
    small_attention_kernel<T, SMAX, RPW><<<grid, 32 * kSmallAttentionWarps, 0, stream>>>(qkv, mask, context, seq, heads, \
                                                                                         hidden, scale)
    if (seq <= 32) {
        if (two_rows) SMALL_ATTENTION(32, 2); else SMALL_ATTENTION(32, 1);
    } else {
        if (two_rows) SMALL_ATTENTION(64, 2); else SMALL_ATTENTION(64, 1);
    }
#undef SMALL_ATTENTION
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

int cubk_attention_small_f32(const float *qkv, const int8_t *mask, int batch, int seq, int heads, int hidden, float scale,
                             float *context, void *stream) {
    return cubk::small_attention<float>(qkv, mask, batch, seq, heads, hidden, scale, context, (cudaStream_t) stream);
}

int cubk_attention_small_f16(const void *qkv, const int8_t *mask, int batch, int seq, int heads, int hidden, float scale,
                             void *context, void *stream) {
    return cubk::small_attention<__half>((const __half *) qkv, mask, batch, seq, heads, hidden, scale, (__half *) context,
                                         (cudaStream_t) stream);
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
