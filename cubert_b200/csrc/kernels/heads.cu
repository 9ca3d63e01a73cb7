// K5b (mean pooling over the sequence axis), K5c (classifier head: logits + bias + softmax)
// and the plain embedding-row gather. K5a (bias + tanh) lives in elementwise.cu.
//
// These touch at most a few MB per call and are latency-bound, except the mean pooler on
// long sequences ([batch, 512, 1024] is 1 MB per sequence), which is a streaming read.
#include <atomic>

#include "common.cuh"

namespace cubk {

// ------------------------------------------------------------------ K5b mean pool
// Block = (32 column vectors) x (BY sequence lanes). Each thread sums every BY-th position
// of its 16-byte column vector inside the block's slice of the sequence; the BY partial sums
// are combined through shared memory. With `splits` > 1 the slices of one sequence go to
// different blocks, which keeps every SM busy when batch * hidden alone is too small a grid:
// each block leaves its float32 partial sums in scratch [batch, splits, hidden] and takes a
// ticket from a counter per (sequence, column block); the block that draws the last ticket adds
// the slices up, always in slice order (so the result does not depend on which block came last),
// and writes the means. Nobody waits for anybody. The counters sit behind the partial sums in
// scratch and are cleared by a memset node in front of the kernel.
constexpr int kPoolBX = 32;
constexpr int kPoolBY = 8;
constexpr int kPoolUnroll = 4;
// The narrow layout: 8 column vectors x 32 sequence lanes per block (a warp reads four rows of 128 bytes).
// Four times the blocks for the same tensor, so that a mid-sized batch fills the GPU without slicing the sequence.
constexpr int kPoolNarrowBX = 8;
constexpr int kPoolNarrowBY = 32;

// Compiled for eight resident blocks per SM (at most 32 registers): the grids this is launched with, up to
// 8 * 148 blocks, then run as ONE wave; with six resident blocks 1024 blocks took 1.15 waves, i.e. two.
template <typename T, int BX, int BY, bool SPLIT>
__global__ void __launch_bounds__(BX *BY, 8)
mean_pool_kernel(const T *x, T *out, float *partial, unsigned int *tickets, int seq, int hidden, int nvec, int splits,
                 int chunk) {
    constexpr int EPV = Vec<T>::EPV;
    __shared__ float smem[BY][BX][EPV + 1];
    __shared__ unsigned int s_ticket;

    const int cv = blockIdx.x * BX + threadIdx.x;
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
        for (int s0 = s_begin + threadIdx.y; s0 < s_end; s0 += BY * kPoolUnroll) {
            uint4 raw[kPoolUnroll];
#pragma unroll
            for (int u = 0; u < kPoolUnroll; ++u) {
                const int s = s0 + u * BY;
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
    const bool writer = threadIdx.y == 0 && cv < nvec;
    if (writer) {
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            float t = 0.f;
#pragma unroll
            for (int y = 0; y < BY; ++y) {
                t += smem[y][threadIdx.x][e];
            }
            acc[e] = t;
        }
    }
    if (SPLIT) {
        if (writer) {
            float4 *dst = reinterpret_cast<float4 *>(partial + ((size_t) b * splits + split) * hidden + (size_t) cv * EPV);
#pragma unroll
            for (int q = 0; q < EPV / 4; ++q) {
                dst[q] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
            }
            __threadfence();  // this thread's partial sums are visible before the block's ticket is drawn
        }
        __syncthreads();
        if (threadIdx.x == 0 && threadIdx.y == 0) {
            s_ticket = atomicAdd(&tickets[(size_t) b * gridDim.x + blockIdx.x], 1u);
        }
        __syncthreads();
        if (s_ticket != (unsigned int) splits - 1) {
            return;  // other slices of this sequence are still on their way; the last one finishes
        }
        __threadfence();
        if (writer) {
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                acc[e] = 0.f;
            }
            for (int k = 0; k < splits; ++k) {
                const float4 *src =
                    reinterpret_cast<const float4 *>(partial + ((size_t) b * splits + k) * hidden + (size_t) cv * EPV);
#pragma unroll
                for (int q = 0; q < EPV / 4; ++q) {
                    const float4 f = __ldcg(src + q);  // from L2: written by other SMs
                    acc[4 * q] += f.x;
                    acc[4 * q + 1] += f.y;
                    acc[4 * q + 2] += f.z;
                    acc[4 * q + 3] += f.w;
                }
            }
        }
    }
    if (writer) {
        float m[EPV];
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            m[e] = acc[e] / (float) seq;
        }
        st_vec(out + (size_t) b * hidden + (size_t) cv * EPV, Vec<T>::pack(m));
    }
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

// Blocks wanted in flight: four per SM on 148 SMs (half of what fits; measured at [64, 512, 1024] binary16,
// two waves of 148 left the GPU half empty).
constexpr int64_t kPoolWantBlocks = 4 * 148;

// Whether the narrow layout is the one to use: the wide one would leave the GPU under-filled and the narrow
// one fills it without slicing the sequence.
static bool mean_pool_narrow(int batch, int seq, int nvec) {
    const int64_t wide = (int64_t) batch * ((nvec + kPoolBX - 1) / kPoolBX);
    const int64_t narrow = (int64_t) batch * ((nvec + kPoolNarrowBX - 1) / kPoolNarrowBX);
    return wide < kPoolWantBlocks && narrow >= kPoolWantBlocks && seq >= 4 * kPoolNarrowBY;
}

// Number of sequence slices (wide layout): 1 when batch * column blocks already gives the blocks wanted or the
// narrow layout does, otherwise enough slices to get there, each at least 32 positions long.
static int mean_pool_splits(int batch, int seq, int hidden, int epv) {
    if (hidden % epv != 0) {
        return 1;
    }
    const int nvec = hidden / epv;
    const int64_t blocks = (int64_t) batch * ((nvec + kPoolBX - 1) / kPoolBX);
    const int64_t want = kPoolWantBlocks;
    if (blocks >= want || seq < 64 || mean_pool_narrow(batch, seq, nvec)) {
        return 1;
    }
    int64_t splits = (want + blocks - 1) / blocks;
    const int64_t max_splits = seq / 32;
    if (splits > max_splits) {
        splits = max_splits;
    }
    return splits < 1 ? 1 : (int) splits;
}

// Bytes of the partial sums (a multiple of 16) and of the ticket counters behind them.
static size_t pool_partial_bytes(int batch, int splits, int hidden) {
    return sizeof(float) * (size_t) batch * splits * hidden;
}

static size_t pool_ticket_bytes(int batch, int nvec) {
    return (sizeof(unsigned int) * (size_t) batch * ((nvec + kPoolBX - 1) / kPoolBX) + 15) / 16 * 16;
}

// Whether the vector kernel (the only one that splits, hence the only one that needs scratch) takes the call.
template <typename T>
static bool mean_pool_vectorised(const void *x, const void *out, int batch, int hidden) {
    return hidden % Vec<T>::EPV == 0 && (x == nullptr || aligned16(x)) && (out == nullptr || aligned16(out)) &&
           batch <= 65535;
}

template <typename T>
size_t mean_pool_scratch_bytes(int batch, int seq, int hidden) {
    if (batch <= 0 || seq <= 0 || hidden <= 0 || !mean_pool_vectorised<T>(nullptr, nullptr, batch, hidden)) {
        return 0;
    }
    const int splits = mean_pool_splits(batch, seq, hidden, Vec<T>::EPV);
    return splits == 1 ? 0 : pool_partial_bytes(batch, splits, hidden) + pool_ticket_bytes(batch, hidden / Vec<T>::EPV);
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
    if (!mean_pool_vectorised<T>(x, out, batch, hidden)) {
        const int64_t n = (int64_t) batch * hidden;
        mean_pool_generic_kernel<T><<<(unsigned) ((n + 255) / 256), 256, 0, stream>>>(x, out, batch, seq, hidden);
        return check_launch();
    }
    const int nvec = hidden / EPV;
    const int splits = mean_pool_splits(batch, seq, hidden, EPV);
    unsigned int *tickets = nullptr;
    if (splits > 1) {
        const size_t partial_bytes = pool_partial_bytes(batch, splits, hidden);
        const size_t ticket_bytes = pool_ticket_bytes(batch, nvec);
        if (scratch == nullptr || scratch_bytes < partial_bytes + ticket_bytes || !aligned16(scratch)) {
            return CUBK_ERR_SCRATCH;
        }
        tickets = reinterpret_cast<unsigned int *>(static_cast<char *>(scratch) + partial_bytes);
        const cudaError_t err = cudaMemsetAsync(tickets, 0, ticket_bytes, stream);
        if (err != cudaSuccess) {
            set_last_error(err);
            return CUBK_ERR_LAUNCH;
        }
    }
    const int chunk = (seq + splits - 1) / splits;
    if (splits == 1 && mean_pool_narrow(batch, seq, nvec)) {
        const dim3 grid((nvec + kPoolNarrowBX - 1) / kPoolNarrowBX, 1, batch);
        mean_pool_kernel<T, kPoolNarrowBX, kPoolNarrowBY, false><<<grid, dim3(kPoolNarrowBX, kPoolNarrowBY), 0, stream>>>(
            x, out, nullptr, nullptr, seq, hidden, nvec, 1, chunk);
        return check_launch();
    }
    const dim3 grid((nvec + kPoolBX - 1) / kPoolBX, splits, batch);
    if (splits > 1) {
        mean_pool_kernel<T, kPoolBX, kPoolBY, true><<<grid, dim3(kPoolBX, kPoolBY), 0, stream>>>(
            x, out, (float *) scratch, tickets, seq, hidden, nvec, splits, chunk);
    } else {
        mean_pool_kernel<T, kPoolBX, kPoolBY, false><<<grid, dim3(kPoolBX, kPoolBY), 0, stream>>>(
            x, out, nullptr, nullptr, seq, hidden, nvec, 1, chunk);
    }
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
// device current. A slot is written once; threads that race to fill it store the same value.
static std::atomic<void *> g_static_pool_scratch_addr[kMaxDevices];

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
    void *p = g_static_pool_scratch_addr[device].load(std::memory_order_relaxed);
    if (p == nullptr) {
        err = cudaGetSymbolAddress(&p, g_static_pool_scratch);
        if (err != cudaSuccess || p == nullptr) {
            set_last_error(err);
            return CUBK_ERR_LAUNCH;
        }
        g_static_pool_scratch_addr[device].store(p, std::memory_order_relaxed);
    }
    *addr = p;
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

// ------------------------------------------------------------------ K5a + K5c in one launch
// pooled = tanh(x + pooler_bias) written out, then the classifier on it: what bias_act_kernel<Tanh>
// followed by logits_probs_kernel computes, for the small label counts of a classification head.
// One 128-thread block per sequence; a thread owns whole 16-byte vectors of the row (all its reads
// of x, the pooler bias and the classifier rows are 128-bit), keeps its slice of the pooled row in
// registers -- in storage precision, since the reference's classifier reads the stored pooled
// output -- and accumulates the dot products of up to kHeadLabels labels at once, which one block
// reduction then finishes. Saves a launch (and a round trip of the pooled row) on the path that
// bounds small-batch serving.
constexpr int kHeadLabels = 8;        // label rows handled per launch
constexpr int kHeadMaxVectors = 4;    // vectors per thread: rows up to 128 * 4 vectors

// POOLER = false: x is the pooled row already (no bias, no tanh, nothing stored back): the classifier alone
// for small label counts, which is how cubk_logits_probs_* runs them.
template <typename T, bool POOLER>
__global__ void __launch_bounds__(128)
pooler_head_kernel(const T *x, const T *pooler_bias, const T *weights, const T *bias, int hidden, int nvec, int labels,
                   T *pooled, T *logits, T *probs) {
    constexpr int EPV = Vec<T>::EPV;
    __shared__ float red[4][kHeadLabels];
    __shared__ float s_logits[kHeadLabels];
    const int b = blockIdx.x;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    float acc[kHeadLabels];
#pragma unroll
    for (int l = 0; l < kHeadLabels; ++l) {
        acc[l] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < kHeadMaxVectors; ++k) {
        const int idx = threadIdx.x + k * 128;
        if (idx < nvec) {
            float v[EPV];
            Vec<T>::unpack(ld_stream(x + (size_t) b * hidden + (size_t) idx * EPV), v);
            if (POOLER) {
                float pb[EPV];
                Vec<T>::unpack(ld_param(pooler_bias + (size_t) idx * EPV), pb);
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    v[e] = tanhf(v[e] + pb[e]);
                }
                const uint4 stored = Vec<T>::pack(v);
                st_vec(pooled + (size_t) b * hidden + (size_t) idx * EPV, stored);
                Vec<T>::unpack(stored, v);  // what the classifier sees is the stored pooled output
            }
#pragma unroll
            for (int l = 0; l < kHeadLabels; ++l) {
                if (l < labels) {
                    float w[EPV];
                    Vec<T>::unpack(ld_param(weights + (size_t) l * hidden + (size_t) idx * EPV), w);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        acc[l] = fmaf(w[e], v[e], acc[l]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int l = 0; l < kHeadLabels; ++l) {
        acc[l] = group_sum<32>(acc[l]);
        if (lane == 0) {
            red[warp][l] = acc[l];
        }
    }
    __syncthreads();
    if (threadIdx.x < labels) {
        const int l = threadIdx.x;
        float t = (red[0][l] + red[1][l]) + (red[2][l] + red[3][l]);
        if (bias != nullptr) {
            t = to_float<T>(bias[l]) + t;
        }
        const T stored = from_float<T>(t);  // the softmax reads the stored logit (op_out/AdditionalOutputLayer.cpp:61-64)
        logits[(size_t) b * labels + l] = stored;
        s_logits[l] = to_float<T>(stored);
    }
    if (probs == nullptr) {
        return;
    }
    __syncthreads();
    if (threadIdx.x < labels) {
        float mx = s_logits[0];
        for (int l = 1; l < labels; ++l) {
            mx = fmaxf(mx, s_logits[l]);
        }
        float sum = 0.f;
        for (int l = 0; l < labels; ++l) {
            sum += expf(s_logits[l] - mx);
        }
        probs[(size_t) b * labels + threadIdx.x] = from_float<T>(expf(s_logits[threadIdx.x] - mx) / sum);
    }
}

// CUBK_ERR_UNSUPPORTED tells the caller to use cubk_bias_tanh_* and cubk_logits_probs_* instead.
template <typename T>
int pooler_head(const T *x, const T *pooler_bias, const T *weights, const T *bias, int batch, int hidden, int labels,
                T *pooled, T *logits, T *probs, cudaStream_t stream) {
    if (x == nullptr || pooler_bias == nullptr || weights == nullptr || pooled == nullptr || logits == nullptr ||
        batch < 0 || hidden <= 0 || labels <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    constexpr int EPV = Vec<T>::EPV;
    if (labels > kHeadLabels || hidden % EPV != 0 || hidden / EPV > 128 * kHeadMaxVectors || !aligned16(x) ||
        !aligned16(pooler_bias) || !aligned16(weights) || !aligned16(pooled)) {
        return CUBK_ERR_UNSUPPORTED;
    }
    if (batch == 0) {
        return CUBK_OK;
    }
    pooler_head_kernel<T, true><<<batch, 128, 0, stream>>>(x, pooler_bias, weights, bias, hidden, hidden / EPV, labels,
                                                           pooled, logits, probs);
    return check_launch();
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
    constexpr int EPV = Vec<T>::EPV;
    if (labels <= kHeadLabels && hidden % EPV == 0 && hidden / EPV <= 128 * kHeadMaxVectors && aligned16(pooled) &&
        aligned16(weights)) {
        // few labels: 128-bit loads and every thread on every label (the kernel of cubk_pooler_head_* without
        // its pooler part); 2 labels, hidden 768, 256 sequences: 11 us with the kernel below
        pooler_head_kernel<T, false><<<batch, 128, 0, stream>>>(pooled, nullptr, weights, bias, hidden, hidden / EPV,
                                                                labels, nullptr, logits, probs);
        return check_launch();
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
    if ((elem_bytes != 2 && elem_bytes != 4) || x == nullptr || out == nullptr || batch < 0 || seq <= 0 || hidden <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    // scratch is needed exactly when the ordinary entry point would take its split path for these operands
    size_t need = 0;
    if (elem_bytes == 4 ? cubk::mean_pool_vectorised<float>(x, out, batch, hidden)
                        : cubk::mean_pool_vectorised<__half>(x, out, batch, hidden)) {
        need = elem_bytes == 4 ? cubk::mean_pool_scratch_bytes<float>(batch, seq, hidden)
                               : cubk::mean_pool_scratch_bytes<__half>(batch, seq, hidden);
    }
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

int cubk_pooler_head_f32(const float *x, const float *pooler_bias, const float *weights, const float *bias, int batch,
                         int hidden, int labels, float *pooled, float *logits, float *probs, void *stream) {
    return cubk::pooler_head<float>(x, pooler_bias, weights, bias, batch, hidden, labels, pooled, logits, probs,
                                    (cudaStream_t) stream);
}

int cubk_pooler_head_f16(const void *x, const void *pooler_bias, const void *weights, const void *bias, int batch,
                         int hidden, int labels, void *pooled, void *logits, void *probs, void *stream) {
    return cubk::pooler_head<__half>((const __half *) x, (const __half *) pooler_bias, (const __half *) weights,
                                     (const __half *) bias, batch, hidden, labels, (__half *) pooled,
                                     (__half *) logits, (__half *) probs, (cudaStream_t) stream);
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
