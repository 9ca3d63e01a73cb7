// K5b (mean pooling over the sequence axis), K5c (classifier head: logits + bias + softmax)
// and the plain embedding-row gather. K5a (bias + tanh) lives in elementwise.cu.
//
// These touch at most a few MB per call and are latency-bound, except the mean pooler on
// long sequences ([batch, 512, 1024] is 1 MB per sequence), which is a streaming read.
#include "common.cuh"

namespace cubk {

// ------------------------------------------------------------------ K5b mean pool
// Block = (32 column vectors) x (BY sequence lanes). Each thread sums every BY-th position
// of its 16-byte column vector inside the block's slice of the sequence; the BY partial sums
// are combined through shared memory. With `splits` > 1 the slices of one sequence go to
// different blocks, which leave float32 partial sums in scratch [batch, splits, hidden] for
// mean_pool_finish_kernel; that keeps every SM busy when batch * hidden alone is too small
// a grid.
constexpr int kPoolBX = 32;
constexpr int kPoolBY = 8;
constexpr int kPoolUnroll = 4;

template <typename T>
__global__ void __launch_bounds__(kPoolBX *kPoolBY)
mean_pool_kernel(const T *x, T *out, float *partial, int seq, int hidden, int nvec, int splits, int chunk) {
    constexpr int EPV = Vec<T>::EPV;
    __shared__ float smem[kPoolBY][kPoolBX][EPV + 1];

    const int cv = blockIdx.x * kPoolBX + threadIdx.x;
    const int split = blockIdx.y;
    const int b = blockIdx.z;
    const int s_begin = split * chunk;
    const int s_end = min(seq, s_begin + chunk);

    float acc[EPV];
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
        acc[e] = 0.f;
    }
    if (cv < nvec) {
        const T *base = x + ((size_t) b * seq) * hidden + (size_t) cv * EPV;
        for (int s0 = s_begin + threadIdx.y; s0 < s_end; s0 += kPoolBY * kPoolUnroll) {
            uint4 raw[kPoolUnroll];
#pragma unroll
            for (int u = 0; u < kPoolUnroll; ++u) {
                const int s = s0 + u * kPoolBY;
                raw[u] = s < s_end ? ld_stream(base + (size_t) s * hidden) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kPoolUnroll; ++u) {
                float v[EPV];
                Vec<T>::unpack(raw[u], v);
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    acc[e] += v[e];
                }
            }
        }
    }
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
        smem[threadIdx.y][threadIdx.x][e] = acc[e];
    }
    __syncthreads();
    if (threadIdx.y == 0 && cv < nvec) {
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            float t = 0.f;
#pragma unroll
            for (int y = 0; y < kPoolBY; ++y) {
                t += smem[y][threadIdx.x][e];
            }
            acc[e] = t;
        }
        if (splits == 1) {
            T *dst = out + (size_t) b * hidden + (size_t) cv * EPV;
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                dst[e] = from_float<T>(acc[e] / (float) seq);
            }
        } else {
            float *dst = partial + ((size_t) b * splits + split) * hidden + (size_t) cv * EPV;
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                dst[e] = acc[e];
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
mean_pool_finish_kernel(const float *partial, T *out, int batch, int seq, int hidden, int splits) {
    const int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (i >= (int64_t) batch * hidden) {
        return;
    }
    const int b = (int) (i / hidden);
    const int c = (int) (i % hidden);
    float t = 0.f;
    for (int k = 0; k < splits; ++k) {
        t += partial[((size_t) b * splits + k) * hidden + c];
    }
    out[i] = from_float<T>(t / (float) seq);
}

// Scalar version for widths or alignments the vector kernel cannot take: thread per (b, c).
template <typename T>
__global__ void __launch_bounds__(256)
mean_pool_generic_kernel(const T *x, T *out, int batch, int seq, int hidden) {
    const int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (i >= (int64_t) batch * hidden) {
        return;
    }
    const int b = (int) (i / hidden);
    const int c = (int) (i % hidden);
    float t = 0.f;
    for (int s = 0; s < seq; ++s) {
        t += to_float<T>(x[((size_t) b * seq + s) * hidden + c]);
    }
    out[i] = from_float<T>(t / (float) seq);
}

// Number of sequence slices: 1 when batch * column blocks already gives two waves of blocks
// on 148 SMs, otherwise enough slices to get there, each at least 32 positions long.
static int mean_pool_splits(int batch, int seq, int hidden, int epv) {
    if (hidden % epv != 0) {
        return 1;
    }
    const int nvec = hidden / epv;
    const int64_t blocks = (int64_t) batch * ((nvec + kPoolBX - 1) / kPoolBX);
    const int64_t want = 2 * 148;
    if (blocks >= want || seq < 64) {
        return 1;
    }
    int64_t splits = (want + blocks - 1) / blocks;
    const int64_t max_splits = seq / 32;
    if (splits > max_splits) {
        splits = max_splits;
    }
    return splits < 1 ? 1 : (int) splits;
}

template <typename T>
size_t mean_pool_scratch_bytes(int batch, int seq, int hidden) {
    if (batch <= 0 || seq <= 0 || hidden <= 0) {
        return 0;
    }
    const int splits = mean_pool_splits(batch, seq, hidden, Vec<T>::EPV);
    return splits == 1 ? 0 : sizeof(float) * (size_t) batch * splits * hidden;
}

template <typename T>
int mean_pool(const T *x, int batch, int seq, int hidden, T *out, void *scratch, size_t scratch_bytes,
              cudaStream_t stream) {
    if (x == nullptr || out == nullptr || batch < 0 || seq <= 0 || hidden <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (batch == 0) {
        return CUBK_OK;
    }
    constexpr int EPV = Vec<T>::EPV;
    const bool vec_ok = hidden % EPV == 0 && aligned16(x) && batch <= 65535;
    if (!vec_ok) {
        const int64_t n = (int64_t) batch * hidden;
        mean_pool_generic_kernel<T><<<(unsigned) ((n + 255) / 256), 256, 0, stream>>>(x, out, batch, seq, hidden);
        return check_launch();
    }
    const int nvec = hidden / EPV;
    const int splits = mean_pool_splits(batch, seq, hidden, EPV);
    if (splits > 1) {
        const size_t need = sizeof(float) * (size_t) batch * splits * hidden;
        if (scratch == nullptr || scratch_bytes < need || !aligned16(scratch)) {
            return CUBK_ERR_SCRATCH;
        }
    }
    const int chunk = (seq + splits - 1) / splits;
    const dim3 grid((nvec + kPoolBX - 1) / kPoolBX, splits, batch);
    mean_pool_kernel<T><<<grid, dim3(kPoolBX, kPoolBY), 0, stream>>>(x, out, (float *) scratch, seq, hidden, nvec,
                                                                     splits, chunk);
    int rc = check_launch();
    if (rc != CUBK_OK || splits == 1) {
        return rc;
    }
    const int64_t n = (int64_t) batch * hidden;
    mean_pool_finish_kernel<T><<<(unsigned) ((n + 255) / 256), 256, 0, stream>>>((const float *) scratch, out,
                                                                                batch, seq, hidden, splits);
    return check_launch();
}

// ------------------------------------------------------------------ K5b without any allocation
// Some hosts of this library are not allowed to call cudaMalloc at all: code that runs inside a
// region where the CUDA allocator is off limits (a real-time serving loop that forbids calls which
// may take the driver's global lock, a plug-in whose host owns every byte of device memory, a
// sandbox that filters allocation calls). For them the split-sequence mean pool is offered with its
// float32 partial sums in a fixed array that is part of the library image: every GPU that loads the
// library sets aside kStaticPoolScratchBytes until the process exits.
constexpr size_t kStaticPoolScratchBytes = CUBK_STATIC_POOL_SCRATCH_BYTES;  // 512 KiB = 131072 partial sums
static __device__ __align__(256) float g_static_pool_scratch[kStaticPoolScratchBytes / sizeof(float)];

// In host code `g_static_pool_scratch` is only a handle for the runtime, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that
// device current. Entries are written once (racing threads store the same value).
static void *g_static_pool_scratch_addr[kMaxDevices] = {nullptr};

static int static_pool_scratch(void **addr) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        set_last_error(err);
        return CUBK_ERR_LAUNCH;
    }
    if (device < 0 || device >= kMaxDevices) {
        return CUBK_ERR_UNSUPPORTED;
    }
    if (g_static_pool_scratch_addr[device] == nullptr) {
        void *p = nullptr;
        err = cudaGetSymbolAddress(&p, g_static_pool_scratch);
        if (err != cudaSuccess || p == nullptr) {
            set_last_error(err);
            return CUBK_ERR_LAUNCH;
        }
        g_static_pool_scratch_addr[device] = p;
    }
    *addr = g_static_pool_scratch_addr[device];
    return CUBK_OK;
}

// ------------------------------------------------------------------ K5c classifier head
// One 128-thread block per sequence. Warp w computes logits w, w+4, ... as dot products with
// coalesced strided reads (the [labels, hidden] weights stay in L2 across blocks); logits
// are kept in shared memory, then the block does the softmax over them.
constexpr int kMaxLabels = 4096;

template <typename T>
__global__ void __launch_bounds__(128)
logits_probs_kernel(const T *pooled, const T *weights, const T *bias, int hidden, int labels, T *logits,
                    T *probs) {
    extern __shared__ float s_logits[];
    __shared__ float red[4];
    const int b = blockIdx.x;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const T *xrow = pooled + (size_t) b * hidden;

    for (int l = warp; l < labels; l += 4) {
        const T *wrow = weights + (size_t) l * hidden;
        float acc = 0.f;
        for (int c = lane; c < hidden; c += 32) {
            acc = fmaf(to_float<T>(wrow[c]), to_float<T>(xrow[c]), acc);
        }
        acc = group_sum<32>(acc);
        if (lane == 0) {
            if (bias != nullptr) {
                acc = to_float<T>(bias[l]) + acc;
            }
            // What later stages see is the stored (storage-precision) logit, as in the reference,
            // whose softmax reads the logits buffer back (op_out/AdditionalOutputLayer.cpp:61-64).
            const T stored = from_float<T>(acc);
            logits[(size_t) b * labels + l] = stored;
            s_logits[l] = to_float<T>(stored);
        }
    }
    if (probs == nullptr) {
        return;
    }
    __syncthreads();

    float mx = -3.0e38f;
    for (int l = threadIdx.x; l < labels; l += 128) {
        mx = fmaxf(mx, s_logits[l]);
    }
    mx = block_max<4>(mx, red);
    float sum = 0.f;
    for (int l = threadIdx.x; l < labels; l += 128) {
        const float e = expf(s_logits[l] - mx);
        s_logits[l] = e;
        sum += e;
    }
    sum = block_sum<4>(sum, red);
    for (int l = threadIdx.x; l < labels; l += 128) {
        probs[(size_t) b * labels + l] = from_float<T>(s_logits[l] / sum);
    }
}

template <typename T>
int logits_probs(const T *pooled, const T *weights, const T *bias, int batch, int hidden, int labels,
                 T *logits, T *probs, cudaStream_t stream) {
    if (pooled == nullptr || weights == nullptr || logits == nullptr || batch < 0 || hidden <= 0 || labels <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (labels > kMaxLabels) {
        return CUBK_ERR_UNSUPPORTED;
    }
    if (batch == 0) {
        return CUBK_OK;
    }
    logits_probs_kernel<T><<<batch, 128, sizeof(float) * labels, stream>>>(pooled, weights, bias, hidden, labels,
                                                                          logits, probs);
    return check_launch();
}

// ------------------------------------------------------------------ embedding row gather
// out[i, :] = table[ids[i], :] as a bit copy. A warp copies one row with 16-byte accesses
// when the row is a whole number of aligned vectors, otherwise byte by byte.
template <typename IdT>
__global__ void __launch_bounds__(128)
embed_gather_kernel(const IdT *ids, int64_t n, const unsigned char *table, int vocab, int row_bytes,
                    unsigned char *out, int vectorised, uint32_t *status) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t) blockIdx.x * 4 + (threadIdx.x >> 5);
    if (i >= n) {
        return;
    }
    int id = (int) ids[i];
    if (id < 0 || id >= vocab) {
        if (status != nullptr && lane == 0) {
            atomicOr(status, CUBK_STATUS_BAD_TOKEN_ID);
        }
        id = min(max(id, 0), vocab - 1);
    }
    const unsigned char *src = table + (size_t) id * row_bytes;
    unsigned char *dst = out + (size_t) i * row_bytes;
    if (vectorised) {
        for (int o = lane * 16; o < row_bytes; o += 32 * 16) {
            st_vec(dst + o, ld_param(src + o));
        }
    } else {
        for (int o = lane; o < row_bytes; o += 32) {
            dst[o] = src[o];
        }
    }
}

template <typename IdT>
int embed_gather(const IdT *ids, int64_t n, const void *table, int vocab, int width, int elem_bytes, void *out,
                 uint32_t *status, cudaStream_t stream) {
    if (ids == nullptr || table == nullptr || out == nullptr || n < 0 || vocab <= 0 || width <= 0 ||
        (elem_bytes != 2 && elem_bytes != 4)) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (n == 0) {
        return CUBK_OK;
    }
    const int64_t grid = (n + 3) / 4;
    if (grid > 0x7fffffffLL) {
        return CUBK_ERR_UNSUPPORTED;
    }
    const int row_bytes = width * elem_bytes;
    const int vectorised = row_bytes % 16 == 0 && aligned16(table) && aligned16(out);
    embed_gather_kernel<IdT><<<(unsigned) grid, 128, 0, stream>>>(ids, n, (const unsigned char *) table, vocab,
                                                                 row_bytes, (unsigned char *) out, vectorised,
                                                                 status);
    return check_launch();
}

// out[idx[i], :] = in[i, :] as a bit copy: the inverse of the gather, used to put the packed rows of
// the non-padding tokens back into their [batch, seq] places. Rows of `out` that no index names are
// left as they are. Duplicate indices must carry identical rows.
__global__ void __launch_bounds__(128)
scatter_rows_kernel(const int32_t *idx, int64_t n, const unsigned char *in, int row_bytes, unsigned char *out,
                    int rows_out, int vectorised) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t) blockIdx.x * 4 + (threadIdx.x >> 5);
    if (i >= n) {
        return;
    }
    const int row = idx[i];
    if (row < 0 || row >= rows_out) {
        return;  // never write outside the destination
    }
    const unsigned char *src = in + (size_t) i * row_bytes;
    unsigned char *dst = out + (size_t) row * row_bytes;
    if (vectorised) {
        for (int o = lane * 16; o < row_bytes; o += 32 * 16) {
            st_vec(dst + o, ld_stream(src + o));
        }
    } else {
        for (int o = lane; o < row_bytes; o += 32) {
            dst[o] = src[o];
        }
    }
}

}  // namespace cubk

extern "C" {

int cubk_scatter_rows(const int32_t *idx, int64_t n, const void *in, int width, int elem_bytes, void *out,
                      int rows_out, void *stream) {
    if (idx == nullptr || in == nullptr || out == nullptr || n < 0 || width <= 0 || rows_out <= 0 ||
        (elem_bytes != 2 && elem_bytes != 4)) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (n == 0) {
        return CUBK_OK;
    }
    const int64_t grid = (n + 3) / 4;
    if (grid > 0x7fffffffLL) {
        return CUBK_ERR_UNSUPPORTED;
    }
    const int row_bytes = width * elem_bytes;
    const int vectorised = row_bytes % 16 == 0 && cubk::aligned16(in) && cubk::aligned16(out);
    cubk::scatter_rows_kernel<<<(unsigned) grid, 128, 0, (cudaStream_t) stream>>>(
        idx, n, (const unsigned char *) in, row_bytes, (unsigned char *) out, rows_out, vectorised);
    return cubk::check_launch();
}

size_t cubk_mean_pool_scratch_bytes(int batch, int seq, int hidden) {
    // The float32 and binary16 kernels split alike for hidden % 8 == 0; take the larger otherwise.
    const size_t a = cubk::mean_pool_scratch_bytes<float>(batch, seq, hidden);
    const size_t b = cubk::mean_pool_scratch_bytes<__half>(batch, seq, hidden);
    return a > b ? a : b;
}

int cubk_mean_pool_f32(const float *x, int batch, int seq, int hidden, float *out, void *scratch,
                       size_t scratch_bytes, void *stream) {
    return cubk::mean_pool<float>(x, batch, seq, hidden, out, scratch, scratch_bytes, (cudaStream_t) stream);
}

int cubk_mean_pool_f16(const void *x, int batch, int seq, int hidden, void *out, void *scratch,
                       size_t scratch_bytes, void *stream) {
    return cubk::mean_pool<__half>((const __half *) x, batch, seq, hidden, (__half *) out, scratch, scratch_bytes,
                                   (cudaStream_t) stream);
}

int cubk_mean_pool_static_scratch(const void *x, int elem_bytes, int batch, int seq, int hidden, void *out,
                                  void *stream) {
    if (elem_bytes != 2 && elem_bytes != 4) {
        return CUBK_ERR_INVALID_ARG;
    }
    const size_t need = elem_bytes == 4 ? cubk::mean_pool_scratch_bytes<float>(batch, seq, hidden)
                                        : cubk::mean_pool_scratch_bytes<__half>(batch, seq, hidden);
    if (need > cubk::kStaticPoolScratchBytes) {
        return CUBK_ERR_SCRATCH;  // the shape needs more partial sums than the built-in array holds
    }
    void *scratch = nullptr;
    if (need > 0) {
        const int rc = cubk::static_pool_scratch(&scratch);
        if (rc != CUBK_OK) {
            return rc;
        }
    }
    if (elem_bytes == 4) {
        return cubk::mean_pool<float>((const float *) x, batch, seq, hidden, (float *) out, scratch,
                                      cubk::kStaticPoolScratchBytes, (cudaStream_t) stream);
    }
    return cubk::mean_pool<__half>((const __half *) x, batch, seq, hidden, (__half *) out, scratch,
                                   cubk::kStaticPoolScratchBytes, (cudaStream_t) stream);
}

int cubk_logits_probs_f32(const float *pooled, const float *weights, const float *bias, int batch, int hidden,
                          int labels, float *logits, float *probs, void *stream) {
    return cubk::logits_probs<float>(pooled, weights, bias, batch, hidden, labels, logits, probs,
                                     (cudaStream_t) stream);
}

int cubk_logits_probs_f16(const void *pooled, const void *weights, const void *bias, int batch, int hidden,
                          int labels, void *logits, void *probs, void *stream) {
    return cubk::logits_probs<__half>((const __half *) pooled, (const __half *) weights, (const __half *) bias,
                                      batch, hidden, labels, (__half *) logits, (__half *) probs,
                                      (cudaStream_t) stream);
}

int cubk_embed_gather_i32(const int32_t *ids, int64_t n, const void *table, int vocab, int width, int elem_bytes,
                          void *out, uint32_t *status, void *stream) {
    return cubk::embed_gather<int32_t>(ids, n, table, vocab, width, elem_bytes, out, status,
                                       (cudaStream_t) stream);
}

int cubk_embed_gather_i8(const int8_t *ids, int64_t n, const void *table, int vocab, int width, int elem_bytes,
                         void *out, uint32_t *status, void *stream) {
    return cubk::embed_gather<int8_t>(ids, n, table, vocab, width, elem_bytes, out, status,
                                      (cudaStream_t) stream);
}

}
