// K3 (bias + GELU), K5a (bias + tanh) and the two small conversion helpers.
//
// Elementwise over a [rows, channels] matrix with a per-column bias. A thread owns one
// 16-byte column vector and walks down the rows, so its bias stays in registers and
// every warp access is a contiguous 512-byte segment of a row. U independent row loads
// are issued before the first use. HBM traffic: one read and one write of the matrix.
#include "common.cuh"

namespace cubk {

// ------------------------------------------------------------------ activations
// Every activation maps a pair of float32 values, so that the arithmetic can be issued as
// packed .f32x2 instructions.
//
// GELU = x * Phi(x), the reference's x * 0.5 * (1 + erf(x / sqrt(2))) (src/cuBERT/op/GELU.cpp:12-14,
// op/GELU.cu:16-18), evaluated as  max(x, 0) - |x| * Q(|x|)  with the Gaussian tail
// Q(z) = 0.5 * erfc(z / sqrt(2)) = 2^p(z). p is a minimax polynomial fit of log2 Q on [0, 5.6],
// written in w = -z; beyond 5.6 the tail term is below 1e-7 * |x|. There is no cancellation
// for negative x (the reference's 1 + erf loses all digits there) and no branch. Per element:
// one MUFU.EX2, two FMNMX and (DEG + 2) / 2 packed FP32 operations.
//   DEG = 6  : |error| <= 3.2e-5 relative, 15x below half an ulp of binary16 -- binary16 storage
//   DEG = 10 : |error| <= 2.5e-7 relative for x >= 0, 6e-7 of max(|y|, 0.02 |x|) for x < 0 -- float32
template <int DEG>
struct GeluCoef;

template <>
struct GeluCoef<6> {
    static __device__ __forceinline__ float c(int k) {
        constexpr float t[7] = {-1.000034451e+00f, 1.150568843e+00f, -4.604086876e-01f, 5.188094452e-02f,
                                7.448623423e-03f,  6.533698761e-04f, 2.562585178e-05f};
        return t[k];
    }
};

template <>
struct GeluCoef<10> {
    static __device__ __forceinline__ float c(int k) {
        constexpr float t[11] = {-9.999997616e-01f, 1.151114583e+00f,  -4.591476619e-01f, 5.263686553e-02f,
                                 7.207410876e-03f,  1.954334439e-04f,  -1.920824725e-04f, -5.257620796e-05f,
                                 -7.090403869e-06f, -5.148263540e-07f, -1.600383115e-08f};
        return t[k];
    }
};

// max(x, 0) that hands a NaN on (fmaxf would return 0 for it): a NaN that reaches the activation, say
// from a binary16 overflow in the product before it, stays visible in the output as it does in the
// reference's x * 0.5 * (1 + erf(..)).
__device__ __forceinline__ float relu_keep_nan(float x) {
    float y;
    asm("max.NaN.f32 %0, %1, 0f00000000;" : "=f"(y) : "f"(x));
    return y;
}

template <int DEG>
struct GeluTailFit {
    __device__ __forceinline__ float2 operator()(float2 x) const {
        const float2 w = make_float2(fmaxf(-fabsf(x.x), -5.6f), fmaxf(-fabsf(x.y), -5.6f));
        float2 p = splat2(GeluCoef<DEG>::c(DEG));
#pragma unroll
        for (int k = DEG - 1; k >= 0; --k) {
            p = fma2(p, w, splat2(GeluCoef<DEG>::c(k)));
        }
        const float2 q = make_float2(fast_exp2(p.x), fast_exp2(p.y));
        return fma2(w, q, make_float2(relu_keep_nan(x.x), relu_keep_nan(x.y)));
    }
};

struct Tanh {
    __device__ __forceinline__ float2 operator()(float2 x) const {
        return make_float2(tanhf(x.x), tanhf(x.y));
    }
};

// ------------------------------------------------------------------ column-stationary kernel
template <typename T, int BX, int BY, int U, typename Act>
__global__ void __launch_bounds__(BX *BY)
bias_act_kernel(const T *x, const T *bias, T *out, int64_t rows, int channels, int nvec) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    const int cv = blockIdx.x * BX + threadIdx.x;
    if (cv >= nvec) {
        return;
    }
    const Act act;
    float2 b[PAIRS];
    if (bias != nullptr) {
        Vec2<T>::unpack(ld_param(bias + (size_t) cv * EPV), b);
    } else {
#pragma unroll
        for (int e = 0; e < PAIRS; ++e) {
            b[e] = make_float2(0.f, 0.f);
        }
    }
    const int64_t col = (int64_t) cv * EPV;
    const int64_t step = (int64_t) gridDim.y * (BY * U);
    for (int64_t r0 = (int64_t) blockIdx.y * (BY * U) + threadIdx.y; r0 < rows; r0 += step) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t r = r0 + (int64_t) u * BY;
            if (r < rows) {
                raw[u] = ld_stream(x + r * channels + col);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t r = r0 + (int64_t) u * BY;
            if (r < rows) {
                float2 v[PAIRS];
                Vec2<T>::unpack(raw[u], v);
#pragma unroll
                for (int e = 0; e < PAIRS; ++e) {
                    v[e] = act(add2(v[e], b[e]));
                }
                st_vec(out + r * channels + col, Vec2<T>::pack(v));
            }
        }
    }
}

// Any width, any alignment: scalar grid-stride loop.
template <typename T, typename Act>
__global__ void __launch_bounds__(256)
bias_act_generic_kernel(const T *x, const T *bias, T *out, int64_t total, int channels) {
    const Act act;
    const int64_t step = (int64_t) gridDim.x * 256;
    for (int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
        float v = to_float<T>(x[i]);
        if (bias != nullptr) {
            v += to_float<T>(bias[i % channels]);
        }
        out[i] = from_float<T>(act(make_float2(v, 0.f)).x);
    }
}

constexpr int kResidentBlocks = 148 * 8;  // grid cap of the small helper kernels

template <typename T, typename Act>
int bias_act(const T *x, const T *bias, int64_t rows, int channels, T *out, cudaStream_t stream) {
    if (x == nullptr || out == nullptr || rows < 0 || channels <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (rows == 0) {
        return CUBK_OK;
    }
    constexpr int EPV = Vec<T>::EPV;
    constexpr int U = 4;
    const bool vec_ok = channels % EPV == 0 && aligned16(x) && aligned16(out) &&
                        (bias == nullptr || aligned16(bias));
    if (vec_ok) {
        const int nvec = channels / EPV;
        // grid.x covers the columns; grid.y is as many row slices as stay resident together.
#define LAUNCH(BX, BY)                                                                              \
    {                                                                                               \
        static OccupancyCache cache;                                                                \
        auto kernel = bias_act_kernel<T, BX, BY, U, Act>;                                           \
        const int gx = (nvec + BX - 1) / BX;                                                        \
        int64_t gy = (rows + BY * U - 1) / (BY * U);                                                \
        int64_t cap = resident_blocks(kernel, BX * BY, 0, &cache) / gx;                             \
        if (cap < 1) cap = 1;                                                                       \
        if (gy > cap) gy = cap;                                                                     \
        if (gy > 65535) gy = 65535;                                                                 \
        kernel<<<dim3((unsigned) gx, (unsigned) gy), dim3(BX, BY), 0, stream>>>(x, bias, out, rows, \
                                                                                channels, nvec);    \
    }
        if (nvec % 256 == 0) {
            LAUNCH(256, 1);
        } else if (nvec % 128 == 0) {
            LAUNCH(128, 2);
        } else if (nvec % 64 == 0) {
            LAUNCH(64, 4);
        } else {
            LAUNCH(32, 8);
        }
#undef LAUNCH
    } else {
        const int64_t total = rows * (int64_t) channels;
        int64_t grid = (total + 255) / 256;
        if (grid > kResidentBlocks) {
            grid = kResidentBlocks;
        }
        bias_act_generic_kernel<T, Act><<<(unsigned) grid, 256, 0, stream>>>(x, bias, out, total, channels);
    }
    return check_launch();
}

// ------------------------------------------------------------------ helpers
template <typename T>
__global__ void __launch_bounds__(256) not_kernel(const int8_t *in, T *out, int64_t n) {
    const int64_t step = (int64_t) gridDim.x * 256;
    for (int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x; i < n; i += step) {
        out[i] = from_float<T>(in[i] == 0 ? 1.f : 0.f);
    }
}

template <typename T>
int logical_not(const int8_t *in, T *out, int64_t n, cudaStream_t stream) {
    if (in == nullptr || out == nullptr || n < 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (n == 0) {
        return CUBK_OK;
    }
    int64_t grid = (n + 255) / 256;
    if (grid > kResidentBlocks) {
        grid = kResidentBlocks;
    }
    not_kernel<T><<<(unsigned) grid, 256, 0, stream>>>(in, out, n);
    return check_launch();
}

// 8 halves in, two 16-byte float vectors out per step; scalar tail and unaligned fallback.
__global__ void __launch_bounds__(256)
half_to_float_kernel(const __half *in, float *out, int64_t n, int vectorised) {
    const int64_t step = (int64_t) gridDim.x * 256;
    const int64_t tid = (int64_t) blockIdx.x * 256 + threadIdx.x;
    int64_t done = 0;
    if (vectorised) {
        const int64_t nv = n / 8;
        for (int64_t i = tid; i < nv; i += step) {
            float v[8];
            Vec<__half>::unpack(ld_stream(in + i * 8), v);
            st_vec(out + i * 8, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                                           __float_as_uint(v[3])));
            st_vec(out + i * 8 + 4, make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]),
                                               __float_as_uint(v[6]), __float_as_uint(v[7])));
        }
        done = nv * 8;
    }
    for (int64_t i = done + tid; i < n; i += step) {
        out[i] = __half2float(in[i]);
    }
}

}  // namespace cubk

extern "C" {

int cubk_bias_gelu_f32(const float *x, const float *bias, int64_t rows, int channels, float *out, void *stream) {
    return cubk::bias_act<float, cubk::GeluTailFit<10>>(x, bias, rows, channels, out, (cudaStream_t) stream);
}

int cubk_bias_gelu_f16(const void *x, const void *bias, int64_t rows, int channels, void *out, void *stream) {
    return cubk::bias_act<__half, cubk::GeluTailFit<6>>((const __half *) x, (const __half *) bias, rows, channels,
                                                     (__half *) out, (cudaStream_t) stream);
}

int cubk_bias_tanh_f32(const float *x, const float *bias, int64_t rows, int channels, float *out, void *stream) {
    return cubk::bias_act<float, cubk::Tanh>(x, bias, rows, channels, out, (cudaStream_t) stream);
}

int cubk_bias_tanh_f16(const void *x, const void *bias, int64_t rows, int channels, void *out, void *stream) {
    return cubk::bias_act<__half, cubk::Tanh>((const __half *) x, (const __half *) bias, rows, channels,
                                              (__half *) out, (cudaStream_t) stream);
}

int cubk_not_f32(const int8_t *in, float *out, int64_t n, void *stream) {
    return cubk::logical_not<float>(in, out, n, (cudaStream_t) stream);
}

int cubk_not_f16(const int8_t *in, void *out, int64_t n, void *stream) {
    return cubk::logical_not<__half>(in, (__half *) out, n, (cudaStream_t) stream);
}

int cubk_half_to_float(const void *in, float *out, int64_t n, void *stream) {
    if (in == nullptr || out == nullptr || n < 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (n == 0) {
        return CUBK_OK;
    }
    const int vectorised = cubk::aligned16(in) && cubk::aligned16(out);
    int64_t grid = (n / 8 + 255) / 256 + 1;
    if (grid > cubk::kResidentBlocks) {
        grid = cubk::kResidentBlocks;
    }
    cubk::half_to_float_kernel<<<(unsigned) grid, 256, 0, (cudaStream_t) stream>>>((const __half *) in, out, n,
                                                                                  vectorised);
    return cubk::check_launch();
}

}
