// K4: masked, scaled row softmax over attention scores.
//
// v[j] = scale * x[j] + (mask[b, j] == 0 ? -10000 : 0);  out = exp(v - max v) / sum
//
// A row lives in the registers of LPR adjacent lanes (LPR = 1..32, a power of two), VPT
// 16-byte vectors per lane, and every lane group works on ROWS rows at once so that
// ROWS * VPT independent 128-bit loads are in flight per thread. Short rows (seq 32 in
// binary16 is 64 bytes) therefore still produce 512-byte contiguous warp accesses. The
// int8 [batch, seq] mask is read directly (EPV bytes per vector, from L1/L2); the
// reference's score-sized broadcast mask tensor never exists. HBM traffic: one read and
// one write of the score matrix.
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

template <typename T, int LPR, int VPT, int ROWS, int BLOCK>
__global__ void __launch_bounds__(BLOCK)
masked_softmax_kernel(const T *scores, const int8_t *mask, T *out, uint32_t rows, FastDiv rows_per_batch,
                      int seq, int nvec, float scale) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int GPW = 32 / LPR;  // row groups per warp
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR;
    const int l = lane % LPR;
    const uint32_t warp = blockIdx.x * (BLOCK / 32) + (threadIdx.x >> 5);
    const uint64_t first = (uint64_t) warp * (GPW * ROWS);
    if (first >= rows) {
        return;  // whole warp leaves together
    }

    uint4 raw[ROWS][VPT];
    bool live[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const uint64_t row = first + (uint64_t) r * GPW + sub;
        live[r] = row < rows;
        const T *src = scores + row * (uint64_t) seq;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int idx = l + k * LPR;
            raw[r][k] = (live[r] && idx < nvec) ? ld_stream(src + (size_t) idx * EPV) : make_uint4(0, 0, 0, 0);
        }
    }

#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const uint64_t row = first + (uint64_t) r * GPW + sub;
        float v[VPT][EPV];
        float mx = -3.0e38f;
        const int8_t *mask_row = nullptr;
        if (mask != nullptr && live[r]) {
            mask_row = mask + (size_t) fast_div((uint32_t) row, rows_per_batch) * seq;
        }
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int idx = l + k * LPR;
            Vec<T>::unpack(raw[r][k], v[k]);
            if (idx < nvec) {
                if (mask_row != nullptr) {
                    float add[EPV];
                    load_mask_add<T>(mask_row, idx, add);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        v[k][e] = fmaf(scale, v[k][e], add[e]);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        v[k][e] = scale * v[k][e];
                    }
                }
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    mx = fmaxf(mx, v[k][e]);
                }
            }
        }
        mx = group_max<LPR>(mx);

        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            if (l + k * LPR < nvec) {
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    v[k][e] = fast_exp2((v[k][e] - mx) * kLog2e);
                    sum += v[k][e];
                }
            }
        }
        sum = group_sum<LPR>(sum);
        const float inv = 1.f / sum;

        if (live[r]) {
            T *dst = out + row * (uint64_t) seq;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int idx = l + k * LPR;
                if (idx < nvec) {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        v[k][e] *= inv;
                    }
                    st_vec(dst + (size_t) idx * EPV, Vec<T>::pack(v[k]));
                }
            }
        }
    }
}

// Any row length, any alignment: one warp per row, three scalar passes.
template <typename T>
__global__ void __launch_bounds__(128)
masked_softmax_generic_kernel(const T *scores, const int8_t *mask, T *out, int64_t rows, int64_t rows_per_batch,
                              int seq, float scale) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t) blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) {
        return;
    }
    const T *src = scores + row * seq;
    T *dst = out + row * seq;
    const int8_t *mask_row = mask != nullptr ? mask + (row / rows_per_batch) * seq : nullptr;
    float mx = -3.0e38f;
    for (int j = lane; j < seq; j += 32) {
        const float add = (mask_row != nullptr && mask_row[j] == 0) ? kMaskedScore : 0.f;
        mx = fmaxf(mx, fmaf(scale, to_float<T>(src[j]), add));
    }
    mx = group_max<32>(mx);
    float sum = 0.f;
    for (int j = lane; j < seq; j += 32) {
        const float add = (mask_row != nullptr && mask_row[j] == 0) ? kMaskedScore : 0.f;
        sum += fast_exp2((fmaf(scale, to_float<T>(src[j]), add) - mx) * kLog2e);
    }
    sum = group_sum<32>(sum);
    const float inv = 1.f / sum;
    for (int j = lane; j < seq; j += 32) {
        const float add = (mask_row != nullptr && mask_row[j] == 0) ? kMaskedScore : 0.f;
        dst[j] = from_float<T>(fast_exp2((fmaf(scale, to_float<T>(src[j]), add) - mx) * kLog2e) * inv);
    }
}

template <typename T>
int masked_softmax(const T *scores, const int8_t *mask, int64_t rows, int64_t rows_per_batch, int seq,
                   float scale, T *out, cudaStream_t stream) {
    if (scores == nullptr || out == nullptr || rows < 0 || seq <= 0 || (mask != nullptr && rows_per_batch <= 0)) {
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
    const bool vec_ok = seq % EPV == 0 && nvec <= 256 && aligned16(scores) && aligned16(out) &&
                        (mask == nullptr || aligned8(mask)) && rows_per_batch <= 0xffffffffLL;
    if (vec_ok) {
        const FastDiv rpb = make_fastdiv((uint32_t) rows_per_batch);
#define LAUNCH(LPR, VPT, ROWS)                                                                          \
    {                                                                                                   \
        const int64_t rows_per_block = (int64_t) (BLOCK / 32) * (32 / LPR) * ROWS;                      \
        const int64_t grid = (rows + rows_per_block - 1) / rows_per_block;                              \
        masked_softmax_kernel<T, LPR, VPT, ROWS, BLOCK><<<(unsigned) grid, BLOCK, 0, stream>>>(         \
            scores, mask, out, (uint32_t) rows, rpb, seq, nvec, scale);                                 \
    }
        if (nvec <= 1) {
            LAUNCH(1, 1, 4);
        } else if (nvec <= 2) {
            LAUNCH(2, 1, 4);
        } else if (nvec <= 4) {
            LAUNCH(4, 1, 4);
        } else if (nvec <= 8) {
            LAUNCH(8, 1, 4);
        } else if (nvec <= 16) {
            LAUNCH(16, 1, 4);
        } else if (nvec <= 32) {
            LAUNCH(32, 1, 4);
        } else if (nvec <= 64) {
            LAUNCH(32, 2, 2);
        } else if (nvec <= 128) {
            LAUNCH(32, 4, 1);
        } else {
            LAUNCH(32, 8, 1);
        }
#undef LAUNCH
    } else {
        const int64_t grid = (rows + 3) / 4;
        masked_softmax_generic_kernel<T><<<(unsigned) grid, 128, 0, stream>>>(scores, mask, out, rows,
                                                                             rows_per_batch, seq, scale);
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

}
