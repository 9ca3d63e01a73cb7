// Whole attention of short sequences in one launch: scores = scale * Q.K^T, masked softmax, context = P.V
// (src/cuBERT/op_att/AttentionSelf.cpp:96-111, op_att/BatchMatMul.cpp:57-68,124-135, op/Softmax.cpp:19-35), with
// scores and probabilities rounded to the storage type where the reference's three steps store them. Three
// kernels: float32 pipes (any storage type, up to 64 positions), warp-level matrix instructions (binary16, up
// to 128 positions) and tcgen05 with accumulators in tensor memory (binary16, 65 to 128 positions).
#include <atomic>

#include "common.cuh"

namespace cubk {

constexpr float kMaskedScore = -10000.0f;  // src/cuBERT/op_att/AttentionSelf.cpp:58-60
constexpr float kLog2e = 1.4426950408889634f;

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

// float(binary16 pair) + float32 pair without a conversion instruction (add.rn.f32.f16: the binary16 operand
// is widened exactly, one rounding, as convert-then-add); the conversions share the 16-lane pipe of the
// exponentials, which is what paces the softmax of these kernels
__device__ __forceinline__ float2 add_pair_f16(uint32_t packed, float2 c) {
    uint16_t lo, hi;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(packed));
    return make_float2(add_f32_f16(lo, c.x), add_f32_f16(hi, c.y));
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
// Block = one (sequence, head); a warp owns strips of 16 query rows, which it reads as whole 128-byte rows and
// turns into A-operand fragments through a 16-row buffer of its own (the context strip leaves the same way). K and V of the head are staged as binary16 rows of 64 + 8 elements (144 B: the eight
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
    __shared__ __align__(16) __half s_w[SMAX / 16 / STRIPS][16][LD];   // per warp: a Q strip in, a context strip out
    const int b = blockIdx.x / heads;
    const int h = blockIdx.x - b * heads;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const size_t row_stride = 3 * (size_t) hidden;
    const __half *base = qkv + (size_t) b * seq * row_stride + (size_t) h * D;

    // A strip of 16 Q rows is 2 KB: four 16-byte vectors per lane (vector lane + 32 u = chunk (lane & 7) of row
    // lane / 8 + 4 u), read as whole 128-byte rows, passed through this warp's own 16-row buffer and picked up
    // as A-operand fragments by ldmatrix. Rows at and beyond seq are zeros and their results are dropped. The
    // first strip's vectors are in flight during the staging of K and V, the next strip's during the products.
    const int qrow = lane >> 3, qcol = (lane & 7) * 8;
    uint4 qv[4];
    auto load_q = [&](int m0) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = m0 + qrow + 4 * u;
            qv[u] = j < seq ? __ldg(reinterpret_cast<const uint4 *>(base + (size_t) j * row_stride + qcol)) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    load_q(16 * warp);
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
        uint32_t qa[D / 16][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            *reinterpret_cast<uint4 *>(&s_w[warp][qrow + 4 * u][qcol]) = qv[u];
        }
        __syncwarp();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            // tiles: rows 0-7 | rows 8-15 at columns 16 kk, then the same rows at columns 16 kk + 8
            ldmatrix_x4(qa[kk], &s_w[warp][lane & 15][16 * kk + 8 * (lane >> 4)]);
        }
        if (s + 1 < STRIPS) {
            load_q(16 * (warp + WARPS * (s + 1)));
        }
        __syncwarp();   // the buffer is free again: the context strip goes through it below
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
                mma_16x8x16(sc[n], qa[kk], kb[0], kb[1]);
                mma_16x8x16(sc[n + 1], qa[kk], kb[2], kb[3]);
            }
        }

        // masked softmax of rows g and g + 8; a row lives in the four lanes of a quad. The stored score
        // (storage precision), then the additive mask, as K4 reads it.
        float mx0 = -3.0e38f, mx1 = -3.0e38f;
        // (tiles are walked in groups of four, one uniform branch per 32 columns, so that the conversions,
        // exponentials and shared-memory reads of a group overlap; a tile past ext16 inside a group holds
        // zeros and comes out as zeros)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if ((n & 3) == 0 && 8 * n >= ext16) {
                break;
            }
            const int col = 8 * n + 2 * t;
            const float2 madd = *reinterpret_cast<const float2 *>(&s_madd[col]);
            const __half2 h0 = __float22half2_rn(mul2(sc[n][0], scale2));
            const __half2 h1 = __float22half2_rn(mul2(sc[n][1], scale2));
            float2 r0 = add_pair_f16(*reinterpret_cast<const uint32_t *>(&h0), madd);
            float2 r1 = add_pair_f16(*reinterpret_cast<const uint32_t *>(&h1), madd);
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
            if ((n & 3) == 0 && 8 * n >= ext16) {
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
        // the context strip: through the warp's buffer, so that it leaves as whole 128-byte rows
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            *reinterpret_cast<__half2 *>(&s_w[warp][g][8 * n + 2 * t]) = __float22half2_rn(o[n][0]);
            *reinterpret_cast<__half2 *>(&s_w[warp][g + 8][8 * n + 2 * t]) = __float22half2_rn(o[n][1]);
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = m0 + qrow + 4 * u;
            if (j < seq) {
                *reinterpret_cast<uint4 *>(context + ((size_t) b * seq + j) * hidden + (size_t) h * D + qcol) =
                    *reinterpret_cast<const uint4 *>(&s_w[warp][qrow + 4 * u][qcol]);
            }
        }
        __syncwarp();   // before the next strip's Q rows overwrite the buffer
    }
}

// ---- binary16 storage, 65 to 128 positions: the same computation on the fifth-generation tensor cores
// One (sequence, head) is exactly one 128-row tile: S = Q.K^T is a single tcgen05.mma chain (M = 128,
// N = the key extent rounded up to 16, K = 64) with its float32 accumulators in tensor memory; every thread of
// the block's one warpgroup then owns a whole score row (tensor-memory lane = query row), so the masked
// softmax needs no shuffles; the probabilities go back to shared memory as the A operand of the second chain,
// O = P.V (M = 128, N = 64, K = extent), whose accumulators overlay the scores in tensor memory. Scores and
// probabilities are rounded to binary16 where the three-launch path stores them.
//
// Shared memory: Q, K, V and later P (over Q and K) as [16-byte column chunk][row][8 elements], i.e. the
// no-swizzle canonical layout of the matrix descriptors: an 8-row x 16-byte core matrix is 128 contiguous
// bytes, core matrices of the next 8 rows follow at +128 B, those of the next column chunk at +2048 B. Q, K
// and P are K-major operands (leading-dimension offset 2048 along the reduction, stride offset 128 along
// rows); V is read as an MN-major B operand (8 keys x 8 columns per core matrix: offset 128 along the
// reduction, 2048 along the output columns), so nothing is transposed on the way in.
// Tensor memory: 128 columns per block (scores, then the context in the first 64), four blocks per SM.
// Every wait on the MMA barrier is bounded; a block that gives up writes NaN rows, frees its tensor memory
// and returns.
constexpr int kTcRows = 128;                       // query rows = tensor-memory lanes = threads
constexpr int kTcChunkBytes = kTcRows * 16;        // one 16-byte column chunk of all rows
constexpr int kTcMatrixBytes = 8 * kTcChunkBytes;  // 128 rows x 64 binary16
constexpr int kTcTmemCols = 128;
constexpr int kTcSmemBytes = 3 * kTcMatrixBytes + kTcRows * 4 + 64;

__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // start address, leading and stride byte offsets in 16-byte units; descriptor version 1; no swizzle
    return (uint64_t) ((saddr & 0x3ffffu) >> 4) | ((uint64_t) (lbo_bytes >> 4) << 16) | ((uint64_t) (sbo_bytes >> 4) << 32) |
           (1ull << 46);
}

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t) accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_load16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// 32 columns of this thread's lane; no wait: the caller issues what it needs, then waits once
__device__ __forceinline__ void tc_load32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tc_wait_loads() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kTcRows, 4)
attention_tc_kernel(const __half *qkv, const int8_t *mask, __half *context, int seq, int heads, int hidden, float scale) {
    extern __shared__ __align__(128) unsigned char tc_smem[];
    unsigned char *s_q = tc_smem;                         // later: P, chunks 0..7
    unsigned char *s_k = tc_smem + kTcMatrixBytes;        // later: P, chunks 8..15
    unsigned char *s_v = tc_smem + 2 * kTcMatrixBytes;
    float *s_madd = reinterpret_cast<float *>(tc_smem + 3 * kTcMatrixBytes);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(tc_smem + 3 * kTcMatrixBytes + kTcRows * 4);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 1);
    int *s_last = reinterpret_cast<int *>(s_tmem + 1);    // 4 ints
    constexpr int D = kSmallHeadDim;
    const int b = blockIdx.x / heads;
    const int h = blockIdx.x - b * heads;
    const int row = threadIdx.x;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const size_t row_stride = 3 * (size_t) hidden;
    const __half *base = qkv + (size_t) b * seq * row_stride + (size_t) h * D;

    // this thread's Q row, in flight while the mask is read
    // (vector u of this thread: 16-byte chunk (tid & 7) of row (tid >> 3) + 16 u, so that a warp reads four whole
    // 128-byte rows per instruction)
    const int chunk = threadIdx.x & 7;
    const int row8 = threadIdx.x >> 3;
    uint4 q[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int j = row8 + 16 * u;
        q[u] = j < seq ? __ldg(reinterpret_cast<const uint4 *>(base + (size_t) j * row_stride) + chunk) : make_uint4(0u, 0u, 0u, 0u);
    }
    // additive mask terms and the key extent: one past the last kept key (every key when none is kept)
    {
        const bool kept = row < seq && (mask == nullptr || mask[(size_t) b * seq + row] != 0);
        s_madd[row] = kept ? 0.f : kMaskedScore;
        const unsigned ballot = __ballot_sync(0xffffffffu, kept);
        if (lane == 0) {
            s_last[warp] = ballot != 0u ? 32 * warp + 32 - __clz(ballot) : 0;
        }
    }
    // tensor memory and the MMA barrier, once this thread's loads are in flight
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(s_tmem)),
                     "r"((uint32_t) kTcTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (threadIdx.x == 0) {
        mbar_init(s_bar, 1);
        mbar_init_fence();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    int ext;
    {
        const int last = max(max(s_last[0], s_last[1]), max(s_last[2], s_last[3]));
        ext = last > 0 ? last : seq;
    }
    const int ext16 = (ext + 15) & ~15;
    if (row >= ext) {
        s_madd[row] = -1.0e30f;   // a column at or beyond the extent: exp2 gives it exactly 0 (read after the next barrier)
    }
    // this thread's K and V rows: below the extent from memory, up to ext16 zeros, beyond never read. Their
    // loads are issued while the Q row is still in flight (the barrier above waited for the mask only).
    {
        uint4 k[8], v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = row8 + 16 * u;
            const uint4 *kp = reinterpret_cast<const uint4 *>(base + (size_t) j * row_stride + hidden) + chunk;
            k[u] = j < ext ? __ldg(kp) : make_uint4(0u, 0u, 0u, 0u);
            v[u] = j < ext ? __ldg(kp + hidden / 8) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = row8 + 16 * u;
            *reinterpret_cast<uint4 *>(s_q + chunk * kTcChunkBytes + j * 16) = q[u];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = row8 + 16 * u;
            if (j < ext16) {
                *reinterpret_cast<uint4 *>(s_k + chunk * kTcChunkBytes + j * 16) = k[u];
                *reinterpret_cast<uint4 *>(s_v + chunk * kTcChunkBytes + j * 16) = v[u];
            }
        }
    }
    // generic-proxy stores -> visible to the tensor core's reads of shared memory
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // S[128, ext16] = Q . K^T: four steps of 16 along the head dimension (two column chunks each)
    if (threadIdx.x == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t idesc = (1u << 4) | ((uint32_t) (ext16 >> 3) << 17) | ((uint32_t) (kTcRows >> 4) << 24);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t a = tc_smem_desc(smem_addr(s_q) + 2 * kk * kTcChunkBytes, kTcChunkBytes, 128);
            const uint64_t bd = tc_smem_desc(smem_addr(s_k) + 2 * kk * kTcChunkBytes, kTcChunkBytes, 128);
            tc_mma_f16(tmem, a, bd, idesc, kk > 0);
        }
        tc_commit(s_bar);
    }
    bool ok = mbar_wait_bounded(s_bar, 0);
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // masked softmax of this thread's row (tensor-memory lane 32 * warp + lane). One pass over tensor memory:
    // the stored scores (scale * S rounded to binary16) stay in 64 registers, two per register; the additive
    // terms come from shared memory four columns at a time (broadcast reads).
    const uint32_t trow = tmem + ((uint32_t) (32 * warp) << 16);
    const float2 scale2 = splat2(scale);
    const float2 log2e2 = splat2(kLog2e);
    uint32_t sh[kTcRows / 2];
    float mx = -3.0e38f;
#pragma unroll
    for (int c0 = 0; c0 < kTcRows; c0 += 32) {
        if (c0 < ext16) {   // uniform over the block
            uint32_t r[32];
            tc_load32_nowait(trow + c0, r);
            tc_wait_loads();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                // columns the product did not write (the load may reach past ext16) count as zeros; their
                // additive term is -1e30, so they come out as probability 0. No branch inside the 32 columns:
                // conversions, exponentials and shared-memory reads of the group overlap.
                const bool written = c0 + i < ext16;
                const float4 madd = *reinterpret_cast<const float4 *>(&s_madd[c0 + i]);
                const float2 a0 = written ? make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])) : make_float2(0.f, 0.f);
                const float2 a1 = written ? make_float2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])) : make_float2(0.f, 0.f);
                const __half2 h0 = __float22half2_rn(mul2(a0, scale2));
                const __half2 h1 = __float22half2_rn(mul2(a1, scale2));
                sh[(c0 + i) / 2] = *reinterpret_cast<const uint32_t *>(&h0);
                sh[(c0 + i) / 2 + 1] = *reinterpret_cast<const uint32_t *>(&h1);
                const float2 v0 = add_pair_f16(sh[(c0 + i) / 2], make_float2(madd.x, madd.y));
                const float2 v1 = add_pair_f16(sh[(c0 + i) / 2 + 1], make_float2(madd.z, madd.w));
                mx = fmaxf(mx, fmaxf(fmaxf(v0.x, v0.y), fmaxf(v1.x, v1.y)));
            }
        }
    }
    const float2 nm2 = splat2(-mx * kLog2e);
    float2 acc = make_float2(0.f, 0.f);
#pragma unroll
    for (int c0 = 0; c0 < kTcRows; c0 += 4) {
        if ((c0 & ~31) < ext16) {
            const float4 madd = *reinterpret_cast<const float4 *>(&s_madd[c0]);
            const float2 v0 = add_pair_f16(sh[c0 / 2], make_float2(madd.x, madd.y));
            const float2 v1 = add_pair_f16(sh[c0 / 2 + 1], make_float2(madd.z, madd.w));
            const float2 e0 = fma2(v0, log2e2, nm2), e1 = fma2(v1, log2e2, nm2);
            acc = add2(acc, make_float2(fast_exp2(e0.x), fast_exp2(e0.y)));
            acc = add2(acc, make_float2(fast_exp2(e1.x), fast_exp2(e1.y)));
        }
    }
    const float2 inv2 = splat2(1.f / (acc.x + acc.y));
    // the stored probabilities: P takes the place of Q and K (the MMA that read them has completed)
#pragma unroll
    for (int c0 = 0; c0 < kTcRows; c0 += 8) {
        if ((c0 & ~31) < ext16) {
            uint32_t p[4];
#pragma unroll
            for (int i = 0; i < 8; i += 4) {
                const float4 madd = *reinterpret_cast<const float4 *>(&s_madd[c0 + i]);
                const float2 v0 = add_pair_f16(sh[(c0 + i) / 2], make_float2(madd.x, madd.y));
                const float2 v1 = add_pair_f16(sh[(c0 + i) / 2 + 1], make_float2(madd.z, madd.w));
                const float2 e0 = fma2(v0, log2e2, nm2), e1 = fma2(v1, log2e2, nm2);
                const __half2 p0 = __float22half2_rn(mul2(make_float2(fast_exp2(e0.x), fast_exp2(e0.y)), inv2));
                const __half2 p1 = __float22half2_rn(mul2(make_float2(fast_exp2(e1.x), fast_exp2(e1.y)), inv2));
                p[i / 2] = *reinterpret_cast<const uint32_t *>(&p0);
                p[i / 2 + 1] = *reinterpret_cast<const uint32_t *>(&p1);
            }
            // columns c0..c0+7 of this row: chunk c0 / 8 of P
            *reinterpret_cast<uint4 *>(s_q + (c0 / 8) * kTcChunkBytes + row * 16) = make_uint4(p[0], p[1], p[2], p[3]);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();

    // O[128, 64] = P[128, ext16] . V[ext16, 64], accumulators over the first 64 score columns
    if (threadIdx.x == 0 && ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t idesc = (1u << 4) | (1u << 16) | ((uint32_t) (D >> 3) << 17) | ((uint32_t) (kTcRows >> 4) << 24);
        for (int kk = 0; kk < ext16 / 16; ++kk) {
            const uint64_t a = tc_smem_desc(smem_addr(s_q) + 2 * kk * kTcChunkBytes, kTcChunkBytes, 128);
            const uint64_t bd = tc_smem_desc(smem_addr(s_v) + 2 * kk * 128, 128, kTcChunkBytes);
            tc_mma_f16(tmem, a, bd, idesc, kk > 0);
        }
        tc_commit(s_bar);
    }
    ok = ok && mbar_wait_bounded(s_bar, 1);
    ok = __all_sync(0xffffffffu, ok);   // tensor-memory loads are warp-wide
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {
        uint32_t r[2][32];
        if (ok) {
            tc_load32_nowait(trow, r[0]);
            tc_load32_nowait(trow + 32, r[1]);
            tc_wait_loads();
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                r[0][i] = r[1][i] = 0x7fc00000u;   // the block gave up: NaN rows
            }
        }
        // through shared memory (P is no longer read) so that a warp stores four whole 128-byte rows per
        // instruction; a warp re-reads only the 32 rows it wrote itself. Rows of 144 B: conflict-free both ways.
        unsigned char *s_o = s_q;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 8) {
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const __half2 ho = __floats2half2_rn(__uint_as_float(r[c0 / 32][c0 % 32 + i]),
                                                     __uint_as_float(r[c0 / 32][c0 % 32 + i + 1]));
                o[i / 2] = *reinterpret_cast<const uint32_t *>(&ho);
            }
            *reinterpret_cast<uint4 *>(s_o + row * 144 + (c0 / 8) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = 32 * warp + (lane >> 3) + 4 * u;
            if (j < seq) {
                const uint4 val = *reinterpret_cast<const uint4 *>(s_o + j * 144 + (lane & 7) * 16);
                reinterpret_cast<uint4 *>(context + ((size_t) b * seq + j) * hidden + (size_t) h * D)[lane & 7] = val;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t) kTcTmemCols) : "memory");
    }
}

// The kernel's shared memory is above the 48 KB a launch gets without asking: raised once per device.
static int attention_tc_prepare() {
    static std::atomic<uint64_t> prepared{0};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess && dev < 64 && ((prepared.load(std::memory_order_acquire) >> dev) & 1ull) != 0) {
        return CUBK_OK;
    }
    if (err == cudaSuccess) {
        err = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes);
    }
    if (err != cudaSuccess) {
        set_last_error(err);
        return CUBK_ERR_LAUNCH;
    }
    if (dev < 64) {
        prepared.fetch_or(1ull << dev, std::memory_order_release);
    }
    return CUBK_OK;
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
        // 16-byte vectors of Q | K | V and context rows (their strides are multiples of 128 bytes)
        if ((reinterpret_cast<uintptr_t>(qkv) & 15u) == 0 && (reinterpret_cast<uintptr_t>(context) & 15u) == 0) {
            const unsigned blocks = (unsigned) (batch * heads);
            if (seq <= 32) {
                small_attention_mma_kernel<32, 1><<<blocks, 64, 0, stream>>>(qkv, mask, context, seq, heads, hidden, scale);
            } else if (seq <= 64) {
                small_attention_mma_kernel<64, 1><<<blocks, 128, 0, stream>>>(qkv, mask, context, seq, heads, hidden, scale);
            } else if (option(CUBK_OPT_ATTENTION_TENSOR_MEMORY) != 0) {
                const int rc = attention_tc_prepare();
                if (rc != CUBK_OK) {
                    return rc;
                }
                attention_tc_kernel<<<blocks, kTcRows, kTcSmemBytes, stream>>>(qkv, mask, context, seq, heads, hidden, scale);
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

int cubk_attention_small_f32(const float *qkv, const int8_t *mask, int batch, int seq, int heads, int hidden, float scale,
                             float *context, void *stream) {
    return cubk::small_attention<float>(qkv, mask, batch, seq, heads, hidden, scale, context, (cudaStream_t) stream);
}

int cubk_attention_small_f16(const void *qkv, const int8_t *mask, int batch, int seq, int heads, int hidden, float scale,
                             void *context, void *stream) {
    return cubk::small_attention<__half>((const __half *) qkv, mask, batch, seq, heads, hidden, scale, (__half *) context,
                                         (cudaStream_t) stream);
}

}  // extern "C"
