// Shared device/host helpers for the fused BERT layer kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cubert_kernels.h"

namespace cubk {

// ---------------------------------------------------------------- launch status
void set_last_error(cudaError_t err);

// Current value of a CUBK_OPT_* switch (environment default, or what cubk_set_option stored).
int option(int id);

inline int check_launch() {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        set_last_error(err);
        return CUBK_ERR_LAUNCH;
    }
    return CUBK_OK;
}

// Blocks to launch for a persistent (grid-stride) kernel: every SM filled to the occupancy the
// kernel really gets, so that all blocks are resident at once and none forms a ragged tail.
// `cache` is a zero-initialised per-call-site table indexed by device; an entry is reused only
// for the same dynamic shared-memory size (racing writers store equivalent values).
constexpr int kMaxDevices = 64;

struct OccupancyCache {
    int blocks[kMaxDevices];
    size_t smem[kMaxDevices];
};

// With `opt_in`, the kernel is first allowed all the dynamic shared memory the device offers a
// block (needed above 48 KB); the limit is the same for every caller, so racing setters agree.
template <typename Kernel>
inline int resident_blocks(Kernel kernel, int block_threads, size_t dynamic_smem, OccupancyCache *cache,
                           bool opt_in = false) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void) cudaGetLastError();
        return 148;
    }
    if (cache->blocks[device] > 0 && cache->smem[device] == dynamic_smem) {
        return cache->blocks[device];
    }
    if (opt_in) {
        int limit = 0;
        cudaFuncAttributes attr;
        if (cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess ||
            cudaFuncGetAttributes(&attr, kernel) != cudaSuccess ||
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 limit - (int) attr.sharedSizeBytes) != cudaSuccess) {
            (void) cudaGetLastError();
            return 0;  // the launch would be refused: callers fall back
        }
    }
    int sms = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block_threads, dynamic_smem) !=
            cudaSuccess ||
        sms <= 0 || per_sm <= 0) {
        (void) cudaGetLastError();
        return 148;
    }
    cache->smem[device] = dynamic_smem;
    cache->blocks[device] = sms * per_sm;
    return sms * per_sm;
}

inline bool aligned16(const void *p) {
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline bool aligned8(const void *p) {
    return (reinterpret_cast<uintptr_t>(p) & 7u) == 0;
}

// ---------------------------------------------------------------- 16-byte vectors
// One 128-bit global transaction holds EPV elements: 4 floats or 8 halves.
template <typename T>
struct Vec;

template <>
struct Vec<float> {
    static constexpr int EPV = 4;
    static __device__ __forceinline__ void unpack(const uint4 &raw, float (&v)[4]) {
        v[0] = __uint_as_float(raw.x);
        v[1] = __uint_as_float(raw.y);
        v[2] = __uint_as_float(raw.z);
        v[3] = __uint_as_float(raw.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[4]) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                          __float_as_uint(v[3]));
    }
};

template <>
struct Vec<__half> {
    static constexpr int EPV = 8;
    static __device__ __forceinline__ void unpack(const uint4 &raw, float (&v)[8]) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            float2 f = __half22float2(h);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// ---------------------------------------------------------------- packed float32 pairs
// Blackwell executes add/mul/fma on two float32 values with one instruction (.f32x2); the
// kernels below are short of issue slots rather than of FP32 lanes, so halving the
// instruction count of the arithmetic is what buys bandwidth.
#ifdef CUBK_F32X2_ASM
__device__ __forceinline__ uint64_t pack_f2(float2 a) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a.x), "f"(a.y));
    return r;
}
__device__ __forceinline__ float2 unpack_f2(uint64_t r) {
    float2 a;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a.x), "=f"(a.y) : "l"(r));
    return a;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack_f2(a)), "l"(pack_f2(b)), "l"(pack_f2(c)));
    return unpack_f2(d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f2(a)), "l"(pack_f2(b)));
    return unpack_f2(d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f2(a)), "l"(pack_f2(b)));
    return unpack_f2(d);
}
#else
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    return __ffma2_rn(a, b, c);
}

__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    return __fadd2_rn(a, b);
}

__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    return __fmul2_rn(a, b);
}
#endif

__device__ __forceinline__ float2 splat2(float a) {
    return make_float2(a, a);
}

// A 16-byte vector as EPV/2 float pairs.
template <typename T>
struct Vec2;

template <>
struct Vec2<float> {
    static constexpr int PAIRS = 2;
    static __device__ __forceinline__ void unpack(const uint4 &raw, float2 (&v)[2]) {
        v[0] = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
        v[1] = make_float2(__uint_as_float(raw.z), __uint_as_float(raw.w));
    }
    static __device__ __forceinline__ uint4 pack(const float2 (&v)[2]) {
        return make_uint4(__float_as_uint(v[0].x), __float_as_uint(v[0].y), __float_as_uint(v[1].x),
                          __float_as_uint(v[1].y));
    }
};

template <>
struct Vec2<__half> {
    static constexpr int PAIRS = 4;
    static __device__ __forceinline__ void unpack(const uint4 &raw, float2 (&v)[4]) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        }
    }
    static __device__ __forceinline__ uint4 pack(const float2 (&v)[4]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __float22half2_rn(v[i]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// float32 + binary16 in one instruction (PTX add.rn.f32.f16: the binary16 operand is widened exactly,
// the sum is rounded once, as convert-then-add would): v[e] += float(h[e]) for the 8 halves of a vector.
__device__ __forceinline__ float add_f32_f16(uint16_t h, float c) {
    float d;
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(h), "f"(c));
    return d;
}

__device__ __forceinline__ void accumulate_halves(const uint4 &raw, float2 (&v)[4]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint16_t lo, hi;
        asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(w[i]));
        v[i] = make_float2(add_f32_f16(lo, v[i].x), add_f32_f16(hi, v[i].y));
    }
}

// v += float(raw) for one 16-byte vector of storage type T. MIXED picks the one-instruction
// binary16 form above over convert + packed add (same result bit for bit).
template <typename T, bool MIXED>
__device__ __forceinline__ void accumulate_vec(const uint4 &raw, float2 (&v)[Vec2<T>::PAIRS]);

template <>
__device__ __forceinline__ void accumulate_vec<float, false>(const uint4 &raw, float2 (&v)[2]) {
    float2 t[2];
    Vec2<float>::unpack(raw, t);
    v[0] = __fadd2_rn(v[0], t[0]);
    v[1] = __fadd2_rn(v[1], t[1]);
}

template <>
__device__ __forceinline__ void accumulate_vec<float, true>(const uint4 &raw, float2 (&v)[2]) {
    accumulate_vec<float, false>(raw, v);
}

template <>
__device__ __forceinline__ void accumulate_vec<__half, false>(const uint4 &raw, float2 (&v)[4]) {
    float2 t[4];
    Vec2<__half>::unpack(raw, t);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = __fadd2_rn(v[i], t[i]);
    }
}

template <>
__device__ __forceinline__ void accumulate_vec<__half, true>(const uint4 &raw, float2 (&v)[4]) {
    accumulate_halves(raw, v);
}

// Streaming 128-bit load: data that is read once (activations, scores).
__device__ __forceinline__ uint4 ld_stream(const void *p) {
    return __ldcs(reinterpret_cast<const uint4 *>(p));
}

// Read-only cached 128-bit load: small operands every block re-reads (bias, gamma, beta, tables).
__device__ __forceinline__ uint4 ld_param(const void *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
}

__device__ __forceinline__ void st_vec(void *p, const uint4 &v) {
    *reinterpret_cast<uint4 *>(p) = v;
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ float to_float<__half>(__half v) {
    return __half2float(v);
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
    return __float2half_rn(v);
}

// 2^x on the special-function unit: one MUFU.EX2, about 2 ulp, results below 2^-126 flush to 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---------------------------------------------------------------- bulk asynchronous copies (global -> shared)
// The copy engine moves a contiguous run of bytes into shared memory and signals an mbarrier with
// the byte count; no register is held while the data is in flight. Source, destination and size
// must be multiples of 16 bytes. Plain (non-multicast) form only.
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return (uint32_t) __cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// Makes freshly initialised mbarriers visible to the copy engine.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One arrival that also announces `bytes` of copy traffic still to land on the barrier.
__device__ __forceinline__ void mbar_arrive_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_load(void *smem_dst, const void *global_src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(smem_dst)),
                 "l"(__cvta_generic_to_global(global_src)), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Waits for the phase with the given parity to complete. The wait is bounded twice over: by a
// deadline on the GPU's nanosecond timer (kBarrierWaitNs; read every 64 polls, so a wait that
// completes at once never reads it) and by a poll count (which alone bounds the short waits of the
// self-test). Returns false on give-up.
constexpr uint32_t kMaxBarrierPolls = 1u << 22;
constexpr uint64_t kBarrierWaitNs = 200ull * 1000 * 1000;  // 0.2 s: five orders above a copy's latency

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t polls = kMaxBarrierPolls) {
    uint64_t deadline = 0;
    for (uint32_t i = 0; i < polls; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((i & 63u) == 63u) {
            const uint64_t now = global_timer_ns();
            if (deadline == 0) {
                deadline = now + kBarrierWaitNs;
            } else if (now > deadline) {
                return false;
            }
        }
    }
    return false;
}

__device__ __forceinline__ uint4 ld_shared_vec(const void *p) {
    return *reinterpret_cast<const uint4 *>(p);
}

// ---------------------------------------------------------------- reductions
// Butterfly reductions across the WIDTH (power of two, <= 32) adjacent lanes that share a row.
template <int WIDTH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o, 32);
    }
    return v;
}

template <int WIDTH>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o, 32));
    }
    return v;
}

// Sum over all threads of a block of NWARPS warps; every thread gets the result.
// `smem` must hold NWARPS floats and is reusable after the call returns.
template <int NWARPS>
__device__ __forceinline__ float block_sum(float v, float *smem) {
    v = group_sum<32>(v);
    if (NWARPS == 1) {
        return v;
    }
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    __syncthreads();  // protect smem from the previous use
    if (lane == 0) {
        smem[warp] = v;
    }
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
        t += smem[w];
    }
    return t;
}

template <int NWARPS>
__device__ __forceinline__ float block_max(float v, float *smem) {
    v = group_max<32>(v);
    if (NWARPS == 1) {
        return v;
    }
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) {
        smem[warp] = v;
    }
    __syncthreads();
    float t = smem[0];
#pragma unroll
    for (int w = 1; w < NWARPS; ++w) {
        t = fmaxf(t, smem[w]);
    }
    return t;
}

// ---------------------------------------------------------------- unsigned division by a runtime constant
// q = n / d for 32-bit n via one multiply-high and a shift (round-up method).
struct FastDiv {
    uint32_t mul;
    uint32_t shift;
    uint32_t div;
};

inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.div = d;
    if (d == 1) {
        f.mul = 0;
        f.shift = 0;
        return f;
    }
    uint32_t l = 0;
    while ((1ull << l) < d) {
        ++l;
    }
    // m = floor(2^32 * (2^l - d) / d) + 1
    f.mul = (uint32_t) (((1ull << 32) * ((1ull << l) - d)) / d + 1);
    f.shift = l;
    return f;
}

__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv &f) {
    if (f.div == 1) {
        return n;
    }
    uint32_t t = __umulhi(n, f.mul);
    // (t + ((n - t) >> 1)) >> (shift - 1)
    return (t + ((n - t) >> 1)) >> (f.shift - 1);
}

}  // namespace cubk
