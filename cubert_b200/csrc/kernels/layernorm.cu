// K1 (embedding lookup + add + LayerNorm) and K2 (bias + residual + LayerNorm).
//
// Layout of the work
//   * A row lives in registers: TPR threads share a row, each holding VPT 16-byte vectors, so a
//     row is read from HBM exactly once and written once.
//   * For rows that fit one warp, blocks are persistent: the grid is sized to what is resident
//     on the GPU and every row group walks over rows with a grid stride, fetching the next row
//     while it reduces the current one. gamma, beta and bias are converted to float32 once per
//     block and kept in shared memory, laid out so that each 128-bit shared load is
//     conflict-free ([quarter][vector] order). Wider rows take one 128-thread block per row.
//   * Mean and the centred second moment are reduced with warp shuffles (plus one shared-memory
//     hop when a row spans a whole block). Arithmetic is float32, issued as packed .f32x2.
//
// HBM traffic per row: K2 reads x and residual and writes out (3 * C * e bytes);
// K1 reads one gathered word row and writes out (2 * H * e bytes) plus 5 index bytes.
#include "common.cuh"

namespace cubk {

constexpr float kLayerNormEps = 1e-12f;  // src/cuBERT/op/LayerNorm.cpp:35, op/LayerNorm.cu:70

// Warps that gave up waiting for a shared-memory copy since the library was loaded (per device).
__device__ unsigned int g_copy_timeouts = 0;

template <int TPR, int BLOCK>
__device__ __forceinline__ float row_sum(float v, float *red) {
    if (TPR <= 32) {
        return group_sum<TPR>(v);
    } else {
        static_assert(TPR <= 32 || TPR == BLOCK, "a row spans a sub-warp group or the whole block");
        return block_sum<BLOCK / 32>(v, red);
    }
}

// float32 copy of a [channels] parameter in shared memory, as float4 [EPV/4][nvec]: the q-th
// float4 of vector idx sits at [q * nvec + idx].
template <typename T>
__device__ __forceinline__ void stage_param(const T *src, float4 *dst, int nvec, int tid, int nthreads) {
    constexpr int EPV = Vec<T>::EPV;
    for (int idx = tid; idx < nvec; idx += nthreads) {
        float v[EPV];
        if (src != nullptr) {
            Vec<T>::unpack(ld_param(src + (size_t) idx * EPV), v);
        } else {
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                v[e] = 0.f;
            }
        }
#pragma unroll
        for (int q = 0; q < EPV / 4; ++q) {
            dst[q * nvec + idx] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
    }
}

template <typename T>
__device__ __forceinline__ void load_param(const float4 *src, int nvec, int idx, float2 (&p)[Vec2<T>::PAIRS]) {
#pragma unroll
    for (int q = 0; q < Vec<T>::EPV / 4; ++q) {
        const float4 f = src[q * nvec + idx];
        p[2 * q] = make_float2(f.x, f.y);
        p[2 * q + 1] = make_float2(f.z, f.w);
    }
}

// A [channels] parameter as seen by the row kernels: the float32 copy in shared memory (narrow
// rows, persistent blocks) or the original in global memory through the read-only cache (wide
// rows, where three float32 copies would cost too much occupancy).
template <typename T, bool IN_SMEM>
struct Param {
    const float4 *smem;
    const T *global;
    __device__ __forceinline__ void load(int nvec, int idx, float2 (&p)[Vec2<T>::PAIRS]) const {
        if (IN_SMEM) {
            load_param<T>(smem, nvec, idx, p);
        } else {
            Vec2<T>::unpack(ld_param(global + (size_t) idx * Vec<T>::EPV), p);
        }
    }
};

struct NoHook {
    __device__ __forceinline__ void operator()() const {}
};

// Normalise the register-resident row `v` and store it. `after_mean` runs once the first
// reduction has consumed every thread's inputs (the place to recycle the buffer they came from).
template <typename T, int TPR, int VPT, int BLOCK, bool IN_SMEM, typename Hook = NoHook>
__device__ __forceinline__ void normalise_store(float2 (&v)[VPT][Vec2<T>::PAIRS], int lane, int nvec, int channels,
                                                bool active, const Param<T, IN_SMEM> &p_gamma,
                                                const Param<T, IN_SMEM> &p_beta, T *out_row, float *red,
                                                Hook after_mean = Hook()) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        if (lane + k * TPR < nvec) {
#pragma unroll
            for (int e = 0; e < PAIRS; ++e) {
                s2 = add2(s2, v[k][e]);
            }
        }
    }
    const float mean = row_sum<TPR, BLOCK>(s2.x + s2.y, red) / (float) channels;
    const float2 neg_mean = splat2(-mean);
    after_mean();

    float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        if (lane + k * TPR < nvec) {
#pragma unroll
            for (int e = 0; e < PAIRS; ++e) {
                v[k][e] = add2(v[k][e], neg_mean);  // keep the centred value
                q2 = fma2(v[k][e], v[k][e], q2);
            }
        }
    }
    const float var = row_sum<TPR, BLOCK>(q2.x + q2.y, red) / (float) channels;
    const float2 rstd = splat2(1.f / sqrtf(var + kLayerNormEps));

#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int idx = lane + k * TPR;
        if (active && idx < nvec) {
            float2 g[PAIRS], b[PAIRS], o[PAIRS];
            p_gamma.load(nvec, idx, g);
            p_beta.load(nvec, idx, b);
#pragma unroll
            for (int e = 0; e < PAIRS; ++e) {
                o[e] = fma2(mul2(g[e], rstd), v[k][e], b[e]);  // beta + (gamma * rstd) * (t - mean)
            }
            st_vec(out_row + (size_t) idx * EPV, Vec2<T>::pack(o));
        }
    }
}

// ------------------------------------------------------------------ K2
// PERSISTENT: blocks loop over rows with a grid stride, parameters staged in shared memory, and
// the next row's loads are issued before the current row is reduced (twice the bytes in flight
// per warp, which binary16 rows need to cover the HBM latency). Otherwise one row group per
// block step and parameters straight from global memory.
template <typename T, int TPR, int VPT, int BLOCK, bool PERSISTENT>
__global__ void __launch_bounds__(BLOCK)
bias_residual_ln_kernel(const T *x, const T *bias, const T *residual, const T *gamma, const T *beta,
                        T *out, int64_t rows, int channels, int nvec) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    constexpr int GROUPS = BLOCK / TPR;
    extern __shared__ float4 s_params[];
    __shared__ float red[BLOCK / 32];
    Param<T, PERSISTENT> p_gamma{s_params, gamma};
    Param<T, PERSISTENT> p_beta{s_params + (EPV / 4) * nvec, beta};
    Param<T, PERSISTENT> p_bias{s_params + 2 * (EPV / 4) * nvec, bias};

    const int lane = threadIdx.x % TPR;
    const int group = threadIdx.x / TPR;
    const int64_t stride = (int64_t) gridDim.x * GROUPS;

    uint4 rx[VPT], rr[VPT];
    auto issue_loads = [&](int64_t row) {
        const bool ok_row = row < rows;
        const int64_t base = ok_row ? row * (int64_t) channels : 0;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int idx = lane + k * TPR;
            const bool ok = ok_row && idx < nvec;
            rx[k] = ok ? ld_stream(x + base + (int64_t) idx * EPV) : make_uint4(0, 0, 0, 0);
            if (residual != nullptr) {
                rr[k] = ok ? ld_stream(residual + base + (int64_t) idx * EPV) : make_uint4(0, 0, 0, 0);
            }
        }
    };

    // The first row's loads go out before the parameters are staged, so that the two latencies overlap.
    int64_t first = (int64_t) blockIdx.x * GROUPS;
    if (first < rows) {
        issue_loads(first + group);
    }
    if (PERSISTENT) {
        stage_param<T>(gamma, s_params, nvec, threadIdx.x, BLOCK);
        stage_param<T>(beta, s_params + (EPV / 4) * nvec, nvec, threadIdx.x, BLOCK);
        if (bias != nullptr) {
            stage_param<T>(bias, s_params + 2 * (EPV / 4) * nvec, nvec, threadIdx.x, BLOCK);
        }
        __syncthreads();
    }
    for (; first < rows; first += stride) {
        const int64_t row = first + group;
        const bool active = row < rows;
        const int64_t base = active ? row * (int64_t) channels : 0;

        float2 v[VPT][PAIRS];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int idx = lane + k * TPR;
            Vec2<T>::unpack(rx[k], v[k]);
            if (bias != nullptr && idx < nvec) {
                float2 b[PAIRS];
                p_bias.load(nvec, idx, b);
#pragma unroll
                for (int e = 0; e < PAIRS; ++e) {
                    v[k][e] = add2(v[k][e], b[e]);
                }
            }
            if (residual != nullptr) {
                float2 r[PAIRS];
                Vec2<T>::unpack(rr[k], r);
#pragma unroll
                for (int e = 0; e < PAIRS; ++e) {
                    v[k][e] = add2(v[k][e], r[e]);
                }
            }
        }
        // The raw registers are free again: fetch the next row while this one is reduced.
        if (first + stride < rows) {
            issue_loads(row + stride);
        }

        normalise_store<T, TPR, VPT, BLOCK, PERSISTENT>(v, lane, nvec, channels, active, p_gamma, p_beta,
                                                        out + base, red);
    }
}

// ------------------------------------------------------------------ K1
// Tokens are walked position-major (j = s * batch + b): every row group takes a contiguous run of j,
// so the position s it works on changes at most a few times and the position row stays in registers
// as float32 across the run. Per token that leaves one gathered word row (from L2: the table is a
// few tens of MB), one token-type row (L1) and the output row. Token indices are fetched one step
// ahead of the row loads that depend on them.
template <typename T, int TPR, int VPT, int BLOCK>
__global__ void __launch_bounds__(BLOCK)
embed_ln_kernel(const int32_t *ids, const int8_t *segment_ids, const T *word, const T *pos, const T *type,
                const T *gamma, const T *beta, T *out, uint32_t tokens, FastDiv batch_div, int seq, int hidden,
                int nvec, int vocab, int type_vocab, uint32_t *status) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    constexpr int GROUPS = BLOCK / TPR;
    extern __shared__ float4 s_params[];
    __shared__ float red[BLOCK / 32];
    Param<T, true> p_gamma{s_params, gamma};
    Param<T, true> p_beta{s_params + (EPV / 4) * nvec, beta};

    const int lane = threadIdx.x % TPR;
    const int group = threadIdx.x / TPR;

    // even split of the position-major index range over all row groups of the grid
    const uint32_t total_groups = gridDim.x * GROUPS;
    const uint32_t g = blockIdx.x * GROUPS + group;
    const uint32_t share = tokens / total_groups;
    const uint32_t extra = tokens - share * total_groups;
    const uint32_t j_begin = g * share + min(g, extra);
    const uint32_t j_count = share + (g < extra ? 1u : 0u);
    // a row that spans the block needs every thread in every step: iterate to the longest run
    const uint32_t steps = TPR == BLOCK ? share + (extra > 0 ? 1u : 0u) : j_count;

    auto token_of = [&](uint32_t j, uint32_t &s) {
        s = fast_div(j, batch_div);
        return (j - s * batch_div.div) * (uint32_t) seq + s;
    };

    int id = 0, seg = 0;
    auto fetch_indices = [&](uint32_t step) {
        id = 0;
        seg = 0;
        if (step < j_count) {
            uint32_t s;
            const uint32_t token = token_of(j_begin + step, s);
            id = ids[token];
            seg = segment_ids[token];
        }
    };

    fetch_indices(0);
    stage_param<T>(gamma, s_params, nvec, threadIdx.x, BLOCK);
    stage_param<T>(beta, s_params + (EPV / 4) * nvec, nvec, threadIdx.x, BLOCK);
    __syncthreads();

    float2 pos_row[VPT][PAIRS];
    uint32_t cur_s = 0xffffffffu;

    for (uint32_t step = 0; step < steps; ++step) {
        const bool active = step < j_count;
        uint32_t s = 0;
        const uint32_t token = active ? token_of(j_begin + step, s) : 0;
        int wid = id, tid = seg;
        if (active) {
            uint32_t bad = 0;
            if (wid < 0 || wid >= vocab) {
                bad |= CUBK_STATUS_BAD_TOKEN_ID;
                wid = min(max(wid, 0), vocab - 1);
            }
            if (tid < 0 || tid >= type_vocab) {
                bad |= CUBK_STATUS_BAD_SEGMENT_ID;
                tid = min(max(tid, 0), type_vocab - 1);
            }
            if (bad != 0 && status != nullptr && lane == 0) {
                atomicOr(status, bad);
            }
        }
        const T *wrow = word + (size_t) wid * hidden;
        const T *trow = type + (size_t) tid * hidden;

        uint4 rw[VPT], rt[VPT];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int idx = lane + k * TPR;
            const bool ok = active && idx < nvec;
            rw[k] = ok ? ld_param(wrow + (size_t) idx * EPV) : make_uint4(0, 0, 0, 0);
            rt[k] = ok ? ld_param(trow + (size_t) idx * EPV) : make_uint4(0, 0, 0, 0);
        }
        if (active && s != cur_s) {  // uniform within a row group
            cur_s = s;
            const T *prow = pos + (size_t) s * hidden;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int idx = lane + k * TPR;
                const uint4 raw = idx < nvec ? ld_param(prow + (size_t) idx * EPV) : make_uint4(0, 0, 0, 0);
                Vec2<T>::unpack(raw, pos_row[k]);
            }
        }
        fetch_indices(step + 1);

        float2 v[VPT][PAIRS];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            float2 t[PAIRS];
            Vec2<T>::unpack(rw[k], v[k]);
            Vec2<T>::unpack(rt[k], t);
#pragma unroll
            for (int e = 0; e < PAIRS; ++e) {
                v[k][e] = add2(add2(v[k][e], pos_row[k][e]), t[e]);  // (word + pos) + type, the reference's order
            }
        }

        normalise_store<T, TPR, VPT, BLOCK, true>(v, lane, nvec, hidden, active, p_gamma, p_beta,
                                                  out + (size_t) token * hidden, red);
    }
}

// K1 for rows that fit one warp, with the gathered word rows staged through shared memory by the
// copy engine. Every warp owns a ring of DEPTH row slots, each with its own mbarrier; lane d (d <
// DEPTH) owns slot d: it issues one bulk copy of the whole word row per step into its slot and reads
// the token indices of the step after that, so DEPTH rows per warp are in flight while no register
// holds them. A slot is refilled after the mean reduction of the row it held, i.e. once every lane's
// shared-memory reads of it have been consumed. Tokens are walked position-major as above.
// A barrier wait that runs out of polls sets CUBK_STATUS_COPY_TIMEOUT and counts in g_copy_timeouts,
// drains (bounded) the copies the warp still has in flight and ends the warp's work.
constexpr int kBulkBlock = 256;

template <typename T, int VPT, int DEPTH>
__global__ void __launch_bounds__(kBulkBlock, (VPT * Vec<T>::EPV <= 24 ? 3 : (VPT * Vec<T>::EPV <= 32 ? 2 : 1)))
embed_ln_bulk_kernel(const int32_t *ids, const int8_t *segment_ids, const T *word, const T *pos, const T *type,
                     const T *gamma, const T *beta, T *out, uint32_t tokens, FastDiv batch_div, int seq,
                     int hidden, int nvec, int vocab, int type_vocab, uint32_t *status) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    constexpr int TPR = 32;
    constexpr int GROUPS = kBulkBlock / TPR;
    static_assert((DEPTH & (DEPTH - 1)) == 0 && DEPTH <= 32, "DEPTH is a power of two");
    extern __shared__ float4 s_dyn[];
    const uint32_t row_bytes = (uint32_t) hidden * (uint32_t) sizeof(T);
    unsigned char *ring_all = reinterpret_cast<unsigned char *>(s_dyn);
    float4 *s_params = reinterpret_cast<float4 *>(ring_all + (size_t) GROUPS * DEPTH * row_bytes);
    uint64_t *bars_all = reinterpret_cast<uint64_t *>(s_params + 2 * (EPV / 4) * nvec);
    Param<T, true> p_gamma{s_params, gamma};
    Param<T, true> p_beta{s_params + (EPV / 4) * nvec, beta};

    const int lane = threadIdx.x % TPR;
    const int group = threadIdx.x / TPR;
    unsigned char *ring = ring_all + (size_t) group * DEPTH * row_bytes;
    uint64_t *bars = bars_all + group * DEPTH;

    const uint32_t total_groups = gridDim.x * GROUPS;
    const uint32_t g = blockIdx.x * GROUPS + group;
    const uint32_t share = tokens / total_groups;
    const uint32_t extra = tokens - share * total_groups;
    const uint32_t j_begin = g * share + min(g, extra);
    const uint32_t j_count = share + (g < extra ? 1u : 0u);

    auto token_of = [&](uint32_t j, uint32_t &s) {
        s = fast_div(j, batch_div);
        return (j - s * batch_div.div) * (uint32_t) seq + s;
    };

    if (lane < DEPTH) {
        mbar_init(&bars[lane], 1);
        mbar_init_fence();
    }
    __syncwarp();

    // slot owners: indices of the row in the slot (seg_cur) and of the row that follows it there
    int id_next = 0, seg_next = 0, seg_cur = 0;
    auto fetch_next = [&](uint32_t step) {
        if (step < j_count) {
            uint32_t s;
            const uint32_t token = token_of(j_begin + step, s);
            id_next = ids[token];
            seg_next = segment_ids[token];
        }
    };
    auto issue = [&](int slot) {  // copy of word[id_next] into `slot`; its segment id becomes current
        int wid = id_next;
        if (wid < 0 || wid >= vocab) {
            if (status != nullptr) {
                atomicOr(status, CUBK_STATUS_BAD_TOKEN_ID);
            }
            wid = min(max(wid, 0), vocab - 1);
        }
        mbar_arrive_expect(&bars[slot], row_bytes);
        bulk_load(ring + (size_t) slot * row_bytes, word + (size_t) wid * hidden, row_bytes, &bars[slot]);
        seg_cur = seg_next;
    };
    if (lane < DEPTH) {
        fetch_next(lane);
        if ((uint32_t) lane < j_count) {
            issue(lane);
        }
        fetch_next(lane + DEPTH);
    }

    stage_param<T>(gamma, s_params, nvec, threadIdx.x, kBulkBlock);
    stage_param<T>(beta, s_params + (EPV / 4) * nvec, nvec, threadIdx.x, kBulkBlock);
    __syncthreads();

    float2 pos_row[VPT][PAIRS];
    uint32_t cur_s = 0xffffffffu;

    for (uint32_t step = 0; step < j_count; ++step) {
        const int slot = (int) (step % DEPTH);
        const uint32_t parity = (step / DEPTH) & 1u;
        uint32_t s = 0;
        const uint32_t token = token_of(j_begin + step, s);
        int tid = __shfl_sync(0xffffffffu, seg_cur, slot);
        if (tid < 0 || tid >= type_vocab) {
            if (status != nullptr && lane == 0) {
                atomicOr(status, CUBK_STATUS_BAD_SEGMENT_ID);
            }
            tid = min(max(tid, 0), type_vocab - 1);
        }
        const T *trow = type + (size_t) tid * hidden;
        uint4 rt[VPT];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int idx = lane + k * TPR;
            rt[k] = idx < nvec ? ld_param(trow + (size_t) idx * EPV) : make_uint4(0, 0, 0, 0);
        }
        if (s != cur_s) {  // uniform within the warp
            cur_s = s;
            const T *prow = pos + (size_t) s * hidden;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int idx = lane + k * TPR;
                const uint4 raw = idx < nvec ? ld_param(prow + (size_t) idx * EPV) : make_uint4(0, 0, 0, 0);
                Vec2<T>::unpack(raw, pos_row[k]);
            }
        }

        if (!mbar_wait_bounded(&bars[slot], parity)) {
            if (lane == 0) {
                atomicAdd(&g_copy_timeouts, 1u);
                if (status != nullptr) {
                    atomicOr(status, CUBK_STATUS_COPY_TIMEOUT);
                }
            }
            // drain what is still in flight (this row and the up to DEPTH - 1 after it), then give up
            for (uint32_t u = step; u < j_count && u < step + DEPTH; ++u) {
                (void) mbar_wait_bounded(&bars[u % DEPTH], (u / DEPTH) & 1u);
            }
            break;
        }
        const unsigned char *srow = ring + (size_t) slot * row_bytes;
        float2 v[VPT][PAIRS];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int idx = lane + k * TPR;
            const uint4 rw = idx < nvec ? ld_shared_vec(srow + (size_t) idx * 16) : make_uint4(0, 0, 0, 0);
            float2 t[PAIRS];
            Vec2<T>::unpack(rw, v[k]);
            Vec2<T>::unpack(rt[k], t);
#pragma unroll
            for (int e = 0; e < PAIRS; ++e) {
                v[k][e] = add2(add2(v[k][e], pos_row[k][e]), t[e]);  // (word + pos) + type, the reference's order
            }
        }

        auto refill = [&]() {
            if (lane == slot) {
                if (step + DEPTH < j_count) {
                    issue(slot);
                }
                fetch_next(step + 2 * DEPTH);
            }
        };
        normalise_store<T, TPR, VPT, kBulkBlock, true>(v, lane, nvec, hidden, true, p_gamma, p_beta,
                                                       out + (size_t) token * hidden, nullptr, refill);
    }
}

// ------------------------------------------------------------------ K2 / K1 for rows of exactly 32 * VPT vectors
// The shapes BERT runs (hidden 768 and 1024 in either storage type) fill a warp exactly, so these
// kernels carry no per-vector bounds predicate and no zero fill; row addresses are vector pointers
// advanced by a constant; the mean uses a precomputed 1 / channels and the scale one rsqrt
// (MUFU.RSQ, 2 ulp; the reference's GPU body uses rsqrtf as well, op/LayerNorm.cu:70); binary16
// inputs enter the float32 sums through add.f32.f16 (one instruction per element instead of a
// conversion and an add). About half the instructions per row of the general kernels above
// (6.7 M against 13.1 M warp instructions on 32768 x 768 binary16), which is what keeps them on the
// memory roofline when the SM clock drops under the power cap inside a BERT step.
constexpr int kRowsBlock = 256;

template <typename T, int VPT>
__device__ __forceinline__ void normalise_store_row(float2 (&v)[VPT][Vec2<T>::PAIRS], int lane, float inv_channels,
                                                    const float4 *s_gamma, const float4 *s_beta, uint4 *dst) {
    constexpr int PAIRS = Vec2<T>::PAIRS;
    constexpr int NVEC = 32 * VPT;
    float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
#pragma unroll
        for (int e = 0; e < PAIRS; ++e) {
            s2 = add2(s2, v[k][e]);
        }
    }
    const float2 neg_mean = splat2(-group_sum<32>(s2.x + s2.y) * inv_channels);
    float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
#pragma unroll
        for (int e = 0; e < PAIRS; ++e) {
            v[k][e] = add2(v[k][e], neg_mean);  // keep the centred value
            q2 = fma2(v[k][e], v[k][e], q2);
        }
    }
    const float2 rstd = splat2(rsqrtf(fmaf(group_sum<32>(q2.x + q2.y), inv_channels, kLayerNormEps)));
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int idx = lane + 32 * k;
        float2 g[PAIRS], b[PAIRS], o[PAIRS];
        load_param<T>(s_gamma, NVEC, idx, g);
        load_param<T>(s_beta, NVEC, idx, b);
#pragma unroll
        for (int e = 0; e < PAIRS; ++e) {
            o[e] = fma2(mul2(g[e], rstd), v[k][e], b[e]);  // beta + (gamma * rstd) * (t - mean)
        }
        dst[idx] = Vec2<T>::pack(o);
    }
}

// K2: a warp per row, persistent blocks; the next row is requested before the current one is reduced.
template <typename T, int VPT>
__global__ void __launch_bounds__(kRowsBlock)
bias_residual_ln_rows_kernel(const T *x, const T *bias, const T *residual, const T *gamma, const T *beta, T *out,
                             int64_t rows, float inv_channels) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    constexpr int NVEC = 32 * VPT;
    constexpr int WARPS = kRowsBlock / 32;
    constexpr bool MIXED = sizeof(T) == 2;
    extern __shared__ float4 s_params[];
    const float4 *s_gamma = s_params;
    const float4 *s_beta = s_params + (EPV / 4) * NVEC;
    const float4 *s_bias = s_params + 2 * (EPV / 4) * NVEC;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint4 *xv = reinterpret_cast<const uint4 *>(x) + lane;
    const uint4 *rv = reinterpret_cast<const uint4 *>(residual) + lane;
    uint4 *ov = reinterpret_cast<uint4 *>(out);
    const int64_t stride = (int64_t) gridDim.x * WARPS;
    int64_t row = (int64_t) blockIdx.x * WARPS + warp;

    uint4 rx[VPT], rr[VPT];
    auto issue_loads = [&](int64_t r) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            rx[k] = __ldcs(xv + r * NVEC + 32 * k);
            rr[k] = __ldcs(rv + r * NVEC + 32 * k);
        }
    };
    // The first row's loads go out before the parameters are staged, so that the two latencies overlap.
    if (row < rows) {
        issue_loads(row);
    }
    stage_param<T>(gamma, s_params, NVEC, threadIdx.x, kRowsBlock);
    stage_param<T>(beta, s_params + (EPV / 4) * NVEC, NVEC, threadIdx.x, kRowsBlock);
    stage_param<T>(bias, s_params + 2 * (EPV / 4) * NVEC, NVEC, threadIdx.x, kRowsBlock);
    __syncthreads();

    for (; row < rows; row += stride) {
        float2 v[VPT][PAIRS];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            load_param<T>(s_bias, NVEC, lane + 32 * k, v[k]);
            accumulate_vec<T, MIXED>(rx[k], v[k]);  // (x + bias)
            accumulate_vec<T, MIXED>(rr[k], v[k]);  //          + residual
        }
        // The raw registers are free again: fetch the next row while this one is reduced.
        if (row + stride < rows) {
            issue_loads(row + stride);
        }
        normalise_store_row<T, VPT>(v, lane, inv_channels, s_gamma, s_beta, ov + row * NVEC);
    }
}

// K1. Tokens are walked position-major as in embed_ln_kernel (the position row stays in registers
// as float32 while a warp works through sequences at one position); the token-type rows sit in shared
// memory beside gamma and beta (float32, up to kMaxTypeRowsSmem of them); the indices of the next token
// are read while the current row is normalised. The gathered word row is NOT requested ahead: holding a
// second row in registers pushed the kernel past the register budget of three resident blocks per SM, and
// the version that spilled to stay there was slower (20.4 us against 19.4 us on 32768 x 768 binary16).
constexpr int kMaxTypeRowsSmem = 4;

template <typename T, int VPT, int MIN_BLOCKS>
__global__ void __launch_bounds__(kRowsBlock, MIN_BLOCKS)
embed_ln_rows_kernel(const int32_t *ids, const int8_t *segment_ids, const T *word, const T *pos, const T *type,
                     const T *gamma, const T *beta, T *out, uint32_t tokens, uint32_t batch, uint32_t seq, int vocab,
                     int type_vocab, uint32_t *status, float inv_hidden) {
    constexpr int EPV = Vec<T>::EPV;
    constexpr int PAIRS = Vec2<T>::PAIRS;
    constexpr int NVEC = 32 * VPT;
    constexpr int WARPS = kRowsBlock / 32;
    constexpr int PV = (EPV / 4) * NVEC;  // float4 per staged row
    constexpr bool MIXED = sizeof(T) == 2;
    extern __shared__ float4 s_params[];
    const float4 *s_gamma = s_params;
    const float4 *s_beta = s_params + PV;
    const float4 *s_type = s_params + 2 * PV;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint4 *wv = reinterpret_cast<const uint4 *>(word) + lane;
    const uint4 *pv = reinterpret_cast<const uint4 *>(pos) + lane;
    uint4 *ov = reinterpret_cast<uint4 *>(out);

    // even split of the position-major index range j = s * batch + b over all warps of the grid
    const uint32_t total_warps = gridDim.x * WARPS;
    const uint32_t w = blockIdx.x * WARPS + warp;
    const uint32_t share = tokens / total_warps;
    const uint32_t extra = tokens - share * total_warps;
    const uint32_t j_begin = w * share + min(w, extra);
    const uint32_t j_count = share + (w < extra ? 1u : 0u);

    uint32_t s = j_begin / batch;       // position and sequence of the current step; token = b * seq + s
    uint32_t b = j_begin - s * batch;
    int id = 0, seg = 0;                // indices of the current step
    if (j_count > 0) {
        id = ids[b * seq + s];
        seg = segment_ids[b * seq + s];
    }
    stage_param<T>(gamma, s_params, NVEC, threadIdx.x, kRowsBlock);
    stage_param<T>(beta, s_params + PV, NVEC, threadIdx.x, kRowsBlock);
    for (int t = 0; t < type_vocab; ++t) {
        stage_param<T>(type + (size_t) t * (NVEC * EPV), s_params + (2 + t) * PV, NVEC, threadIdx.x, kRowsBlock);
    }
    __syncthreads();

    float2 pos_row[VPT][PAIRS];
    bool new_pos = true;
    for (uint32_t step = 0; step < j_count; ++step) {
        int wid = id, tid = seg;
        uint32_t bad = 0;
        if (wid < 0 || wid >= vocab) {
            bad |= CUBK_STATUS_BAD_TOKEN_ID;
            wid = min(max(wid, 0), vocab - 1);
        }
        if (tid < 0 || tid >= type_vocab) {
            bad |= CUBK_STATUS_BAD_SEGMENT_ID;
            tid = min(max(tid, 0), type_vocab - 1);
        }
        if (bad != 0 && status != nullptr && lane == 0) {
            atomicOr(status, bad);
        }
        uint4 rw[VPT];
        const uint4 *src = wv + (size_t) wid * NVEC;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            rw[k] = __ldg(src + 32 * k);
        }
        if (new_pos) {  // uniform within the warp
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                Vec2<T>::unpack(__ldg(pv + (size_t) s * NVEC + 32 * k), pos_row[k]);
            }
        }
        uint4 *dst = ov + ((size_t) b * seq + s) * NVEC;
        // on to the next step's place, and its indices while this row's loads are in flight
        new_pos = false;
        if (++b == batch) {
            b = 0;
            ++s;
            new_pos = true;
        }
        if (step + 1 < j_count) {
            id = ids[b * seq + s];
            seg = segment_ids[b * seq + s];
        }

        const float4 *s_trow = s_type + tid * PV;
        float2 v[VPT][PAIRS];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            float2 t[PAIRS];
            load_param<T>(s_trow, NVEC, lane + 32 * k, t);
#pragma unroll
            for (int e = 0; e < PAIRS; ++e) {
                v[k][e] = pos_row[k][e];
            }
            accumulate_vec<T, MIXED>(rw[k], v[k]);  // (word + pos)
#pragma unroll
            for (int e = 0; e < PAIRS; ++e) {
                v[k][e] = add2(v[k][e], t[e]);      //             + type, the reference's order
            }
        }
        normalise_store_row<T, VPT>(v, lane, inv_hidden, s_gamma, s_beta, dst);
    }
}

// The give-up path of the bounded barrier wait, on its own: one warp waits for a phase that nothing
// will ever complete (no copy is issued, no thread arrives), runs out of its `polls` and reports it
// the way the staged kernels do. Nothing is in flight, so there is nothing to drain.
__global__ void __launch_bounds__(32) copy_wait_timeout_selftest_kernel(uint32_t polls, uint32_t *status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    __syncwarp();
    if (!mbar_wait_bounded(&bar, 0, polls)) {
        if (threadIdx.x == 0) {
            atomicAdd(&g_copy_timeouts, 1u);
            if (status != nullptr) {
                atomicOr(status, CUBK_STATUS_COPY_TIMEOUT);
            }
        }
    }
}

// ------------------------------------------------------------------ generic rows (any width, any alignment)
// One block per row, three scalar passes over the row (sum, centred squares, write).
template <typename T>
struct ResidualLoader {
    const T *x, *bias, *residual;
    int channels;
    __device__ __forceinline__ float operator()(int64_t row, int c) const {
        const int64_t i = row * (int64_t) channels + c;
        float t = to_float<T>(x[i]);
        if (bias != nullptr) {
            t += to_float<T>(bias[c]);
        }
        if (residual != nullptr) {
            t += to_float<T>(residual[i]);
        }
        return t;
    }
};

template <typename T>
struct EmbedLoader {
    const int32_t *ids;
    const int8_t *segment_ids;
    const T *word, *pos, *type;
    int hidden, seq, vocab, type_vocab;
    uint32_t *status;
    __device__ __forceinline__ float operator()(int64_t row, int c) const {
        int id = ids[row];
        int seg = segment_ids[row];
        uint32_t bad = 0;
        if (id < 0 || id >= vocab) {
            bad |= CUBK_STATUS_BAD_TOKEN_ID;
            id = min(max(id, 0), vocab - 1);
        }
        if (seg < 0 || seg >= type_vocab) {
            bad |= CUBK_STATUS_BAD_SEGMENT_ID;
            seg = min(max(seg, 0), type_vocab - 1);
        }
        if (bad != 0 && status != nullptr && c == 0) {
            atomicOr(status, bad);
        }
        const int s = (int) (row % seq);
        return (to_float<T>(word[(size_t) id * hidden + c]) + to_float<T>(pos[(size_t) s * hidden + c])) +
               to_float<T>(type[(size_t) seg * hidden + c]);
    }
};

template <typename T, typename Loader>
__global__ void __launch_bounds__(128)
generic_ln_kernel(Loader load, const T *gamma, const T *beta, T *out, int channels) {
    __shared__ float smem[4];
    const int64_t row = blockIdx.x;
    float s = 0.f;
    for (int c = threadIdx.x; c < channels; c += 128) {
        s += load(row, c);
    }
    const float mean = block_sum<4>(s, smem) / (float) channels;
    float q = 0.f;
    for (int c = threadIdx.x; c < channels; c += 128) {
        const float d = load(row, c) - mean;
        q += d * d;
    }
    const float var = block_sum<4>(q, smem) / (float) channels;
    const float rstd = 1.f / sqrtf(var + kLayerNormEps);
    for (int c = threadIdx.x; c < channels; c += 128) {
        const float t = load(row, c);
        out[row * (int64_t) channels + c] =
            from_float<T>(to_float<T>(beta[c]) + to_float<T>(gamma[c]) * rstd * (t - mean));
    }
}

// ------------------------------------------------------------------ dispatch
// Picks (threads per row, vectors per thread) for a row of `nvec` 16-byte vectors.
// Rows up to 256 vectors stay inside one warp; up to 1024 vectors use one 128-thread block.
#define CUBK_LN_DISPATCH(NVEC, LAUNCH)                             \
    do {                                                           \
        if ((NVEC) <= 32) { LAUNCH(32, 1, 256, true); }            \
        else if ((NVEC) <= 64) { LAUNCH(32, 2, 256, true); }       \
        else if ((NVEC) <= 96) { LAUNCH(32, 3, 256, true); }       \
        else if ((NVEC) <= 128) { LAUNCH(32, 4, 256, true); }      \
        else if ((NVEC) <= 192) { LAUNCH(32, 6, 256, true); }      \
        else if ((NVEC) <= 256) { LAUNCH(32, 8, 256, true); }      \
        else if ((NVEC) <= 384) { LAUNCH(128, 3, 128, false); }    \
        else if ((NVEC) <= 512) { LAUNCH(128, 4, 128, false); }    \
        else if ((NVEC) <= 768) { LAUNCH(128, 6, 128, false); }    \
        else { LAUNCH(128, 8, 128, false); }                       \
    } while (0)

constexpr int kMaxRowVectors = 1024;
constexpr size_t kMaxParamSmem = 47 * 1024;  // dynamic + static stay below the 48 KB that needs no opt-in

// Whether K1 stages its word rows through shared memory. Measured on B200 (hidden 768): with float32
// rows (3 KB) and 32768 tokens the staged kernel takes 30 us against 33 us, with 4096 tokens 8.4 us
// against 7.6 us, and with binary16 rows (1.5 KB) 25 us against 22 us, where the per-row instruction
// cost rather than the bytes in flight sets the pace. So: rows of 2 KB or more and at least 16384 tokens,
// unless CUBK_OPT_EMBED_STAGED_ROWS forces the choice.
static bool use_bulk_rows(size_t row_bytes, int64_t tokens) {
    const int forced = option(CUBK_OPT_EMBED_STAGED_ROWS);
    if (forced == 0 || forced == 1) {
        return forced == 1;
    }
    return row_bytes >= 2048 && tokens >= 16384;
}

// Launch of the exact-width K2 for one VPT.
template <typename T, int VPT>
void launch_ln_rows(const T *x, const T *bias, const T *residual, const T *gamma, const T *beta, T *out,
                    int64_t rows, int channels, cudaStream_t stream) {
    static OccupancyCache cache;
    const size_t smem = sizeof(float) * 3 * (size_t) channels;
    auto kernel = bias_residual_ln_rows_kernel<T, VPT>;
    int64_t grid = (rows + (kRowsBlock / 32) - 1) / (kRowsBlock / 32);
    const int resident = resident_blocks(kernel, kRowsBlock, smem, &cache);
    if (grid > resident) {
        grid = resident;
    }
    kernel<<<(unsigned) grid, kRowsBlock, smem, stream>>>(x, bias, residual, gamma, beta, out, rows,
                                                          1.f / (float) channels);
}

template <typename T>
int bias_residual_ln(const T *x, const T *bias, const T *residual, const T *gamma, const T *beta,
                     int64_t rows, int channels, T *out, cudaStream_t stream) {
    if (x == nullptr || gamma == nullptr || beta == nullptr || out == nullptr || rows < 0 || channels <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    if (rows == 0) {
        return CUBK_OK;
    }
    if (rows > 0x7fffffffLL) {
        return CUBK_ERR_UNSUPPORTED;
    }
    constexpr int EPV = Vec<T>::EPV;
    const bool vec_ok = channels % EPV == 0 && channels / EPV <= kMaxRowVectors && aligned16(x) && aligned16(out) && aligned16(gamma) && aligned16(beta) &&
                        (bias == nullptr || aligned16(bias)) && (residual == nullptr || aligned16(residual));
    if (vec_ok) {
        const int nvec = channels / EPV;
        if (bias != nullptr && residual != nullptr && nvec % 32 == 0 && option(CUBK_OPT_EXACT_WIDTH_ROWS) != 0) {
            bool launched = true;
#define ROWS(VPT) launch_ln_rows<T, VPT>(x, bias, residual, gamma, beta, out, rows, channels, stream)
            switch (nvec / 32) {
                case 1: ROWS(1); break;
                case 2: ROWS(2); break;
                case 3: ROWS(3); break;
                case 4: ROWS(4); break;
                case 6: ROWS(6); break;
                case 8: ROWS(8); break;
                default: launched = false; break;
            }
#undef ROWS
            if (launched) {
                return check_launch();
            }
        }
#define LAUNCH(TPR, VPT, BLOCK, PERSISTENT)                                                           \
    {                                                                                                 \
        static OccupancyCache cache;                                                                  \
        auto kernel = bias_residual_ln_kernel<T, TPR, VPT, BLOCK, PERSISTENT>;                        \
        const size_t smem = PERSISTENT ? sizeof(float) * 3 * (size_t) channels : 0;                   \
        int64_t grid = (rows + (BLOCK / TPR) - 1) / (BLOCK / TPR);                                    \
        if (PERSISTENT) {                                                                             \
            const int resident = resident_blocks(kernel, BLOCK, smem, &cache);                        \
            if (grid > resident) grid = resident;                                                     \
        }                                                                                             \
        kernel<<<(unsigned) grid, BLOCK, smem, stream>>>(x, bias, residual, gamma, beta, out, rows,   \
                                                          channels, nvec);                            \
    }
        CUBK_LN_DISPATCH(nvec, LAUNCH);
#undef LAUNCH
    } else {
        ResidualLoader<T> loader{x, bias, residual, channels};
        generic_ln_kernel<T, ResidualLoader<T>><<<(unsigned) rows, 128, 0, stream>>>(loader, gamma, beta, out,
                                                                                    channels);
    }
    return check_launch();
}

// Launches the shared-memory-staged K1 when its ring fits; false = not launched (caller falls back).
template <typename T, int VPT, int DEPTH>
bool launch_embed_bulk(const int32_t *ids, const int8_t *segment_ids, const T *word, const T *pos, const T *type,
                       const T *gamma, const T *beta, T *out, int64_t tokens, int batch, int seq, int hidden,
                       int nvec, int vocab, int type_vocab, uint32_t *status, cudaStream_t stream) {
    static OccupancyCache cache;
    constexpr int GROUPS = kBulkBlock / 32;
    auto kernel = embed_ln_bulk_kernel<T, VPT, DEPTH>;
    const size_t smem = (size_t) GROUPS * DEPTH * hidden * sizeof(T) + sizeof(float) * 2 * (size_t) hidden +
                        sizeof(uint64_t) * GROUPS * DEPTH;
    const int resident = resident_blocks(kernel, kBulkBlock, smem, &cache, true);
    if (resident <= 0) {
        return false;
    }
    int64_t grid = (tokens + GROUPS - 1) / GROUPS;
    if (grid > resident) {
        grid = resident;
    }
    kernel<<<(unsigned) grid, kBulkBlock, smem, stream>>>(ids, segment_ids, word, pos, type, gamma, beta, out,
                                                          (uint32_t) tokens, make_fastdiv((uint32_t) batch), seq,
                                                          hidden, nvec, vocab, type_vocab, status);
    return true;
}

template <typename T, int VPT>
bool launch_embed_bulk_depth(const int32_t *ids, const int8_t *segment_ids, const T *word, const T *pos,
                             const T *type, const T *gamma, const T *beta, T *out, int64_t tokens, int batch,
                             int seq, int hidden, int nvec, int vocab, int type_vocab, uint32_t *status,
                             cudaStream_t stream) {
    // four rows in flight per warp while eight such rings stay within 64 KB, else two
    if ((size_t) (kBulkBlock / 32) * 4 * hidden * sizeof(T) <= 64 * 1024) {
        return launch_embed_bulk<T, VPT, 4>(ids, segment_ids, word, pos, type, gamma, beta, out, tokens, batch, seq,
                                            hidden, nvec, vocab, type_vocab, status, stream);
    }
    return launch_embed_bulk<T, VPT, 2>(ids, segment_ids, word, pos, type, gamma, beta, out, tokens, batch, seq,
                                        hidden, nvec, vocab, type_vocab, status, stream);
}

// Launch of the exact-width K1 for one VPT; false = the staged rows do not fit shared memory.
// Rows of three vectors per lane (hidden 768 in binary16) are compiled for three resident blocks per
// SM (79 registers, nothing spilled), rows of four (hidden 1024) for two: 19.4 us on 32768 tokens of 768
// against 26 us with the registers the compiler takes when left alone (136, one block per SM).
template <typename T, int VPT>
bool launch_embed_rows(const int32_t *ids, const int8_t *segment_ids, const T *word, const T *pos, const T *type,
                       const T *gamma, const T *beta, T *out, int64_t tokens, int batch, int seq, int hidden,
                       int vocab, int type_vocab, uint32_t *status, cudaStream_t stream) {
    static OccupancyCache cache;
    const size_t smem = sizeof(float) * (2 + (size_t) type_vocab) * (size_t) hidden;
    if (smem > kMaxParamSmem) {
        return false;
    }
    auto kernel = embed_ln_rows_kernel<T, VPT, (VPT == 3 ? 3 : (VPT == 4 ? 2 : 1))>;
    int64_t grid = (tokens + (kRowsBlock / 32) - 1) / (kRowsBlock / 32);
    const int resident = resident_blocks(kernel, kRowsBlock, smem, &cache);
    if (grid > resident) {
        grid = resident;
    }
    kernel<<<(unsigned) grid, kRowsBlock, smem, stream>>>(ids, segment_ids, word, pos, type, gamma, beta, out,
                                                          (uint32_t) tokens, (uint32_t) batch, (uint32_t) seq, vocab,
                                                          type_vocab, status, 1.f / (float) hidden);
    return true;
}

template <typename T>
int embed_ln(const int32_t *ids, const int8_t *segment_ids, const T *word, const T *pos, const T *type,
             const T *gamma, const T *beta, int batch, int seq, int hidden, int vocab, int type_vocab,
             T *out, uint32_t *status, cudaStream_t stream) {
    if (ids == nullptr || segment_ids == nullptr || word == nullptr || pos == nullptr || type == nullptr ||
        gamma == nullptr || beta == nullptr || out == nullptr || batch < 0 || seq <= 0 || hidden <= 0 ||
        vocab <= 0 || type_vocab <= 0) {
        return CUBK_ERR_INVALID_ARG;
    }
    const int64_t tokens = (int64_t) batch * seq;
    if (tokens == 0) {
        return CUBK_OK;
    }
    if (tokens > 0x7fffffffLL) {
        return CUBK_ERR_UNSUPPORTED;
    }
    constexpr int EPV = Vec<T>::EPV;
    const size_t smem = sizeof(float) * 2 * (size_t) hidden;
    const bool vec_ok = hidden % EPV == 0 && hidden / EPV <= kMaxRowVectors && smem <= kMaxParamSmem &&
                        aligned16(word) && aligned16(pos) && aligned16(type) && aligned16(gamma) &&
                        aligned16(beta) && aligned16(out);
    if (vec_ok) {
        const int nvec = hidden / EPV;
        const FastDiv batch_div = make_fastdiv((uint32_t) batch);
        if (nvec <= 256 && use_bulk_rows(sizeof(T) * (size_t) hidden, tokens)) {  // a row fits one warp
            bool launched = false;
#define BULK(VPT)                                                                                           \
    launched = launch_embed_bulk_depth<T, VPT>(ids, segment_ids, word, pos, type, gamma, beta, out, tokens, \
                                               batch, seq, hidden, nvec, vocab, type_vocab, status, stream)
            if (nvec <= 32) { BULK(1); }
            else if (nvec <= 64) { BULK(2); }
            else if (nvec <= 96) { BULK(3); }
            else if (nvec <= 128) { BULK(4); }
            else if (nvec <= 192) { BULK(6); }
            else { BULK(8); }
#undef BULK
            if (launched) {
                return check_launch();
            }
        }
        // binary16 rows that fill a warp exactly (float32 rows are faster on the kernels above and below:
        // 33 us general / 30 us staged against 40 us on 32768 tokens of hidden 768)
        if constexpr (sizeof(T) == 2) {
          if (nvec % 32 == 0 && type_vocab <= kMaxTypeRowsSmem && option(CUBK_OPT_EXACT_WIDTH_EMBED) != 0) {
            bool launched = false;
#define ROWS(VPT)                                                                                              \
    launched = launch_embed_rows<T, VPT>(ids, segment_ids, word, pos, type, gamma, beta, out, tokens, batch, seq, \
                                         hidden, vocab, type_vocab, status, stream)
            switch (nvec / 32) {
                case 1: ROWS(1); break;
                case 2: ROWS(2); break;
                case 3: ROWS(3); break;
                case 4: ROWS(4); break;
                case 6: ROWS(6); break;
                case 8: ROWS(8); break;
                default: break;
            }
#undef ROWS
            if (launched) {
                return check_launch();
            }
          }
        }
#define LAUNCH(TPR, VPT, BLOCK, PERSISTENT)                                                           \
    {                                                                                                 \
        static OccupancyCache cache;                                                                  \
        auto kernel = embed_ln_kernel<T, TPR, VPT, BLOCK>;                                            \
        int64_t grid = (tokens + (BLOCK / TPR) - 1) / (BLOCK / TPR);                                  \
        const int resident = resident_blocks(kernel, BLOCK, smem, &cache);                            \
        if (grid > resident) grid = resident;                                                         \
        kernel<<<(unsigned) grid, BLOCK, smem, stream>>>(ids, segment_ids, word, pos, type, gamma,    \
                                                          beta, out, (uint32_t) tokens, batch_div,    \
                                                          seq, hidden, nvec, vocab, type_vocab,       \
                                                          status);                                    \
    }
        CUBK_LN_DISPATCH(nvec, LAUNCH);
#undef LAUNCH
    } else {
        EmbedLoader<T> loader{ids, segment_ids, word, pos, type, hidden, seq, vocab, type_vocab, status};
        generic_ln_kernel<T, EmbedLoader<T>><<<(unsigned) tokens, 128, 0, stream>>>(loader, gamma, beta, out,
                                                                                   hidden);
    }
    return check_launch();
}

}  // namespace cubk

extern "C" {

int cubk_copy_timeouts(unsigned int *count) {
    if (count == nullptr) {
        return CUBK_ERR_INVALID_ARG;
    }
    cudaError_t err = cudaMemcpyFromSymbol(count, cubk::g_copy_timeouts, sizeof(unsigned int));
    if (err != cudaSuccess) {
        cubk::set_last_error(err);
        return CUBK_ERR_LAUNCH;
    }
    return CUBK_OK;
}

int cubk_selftest_copy_wait_timeout(unsigned int polls, uint32_t *status, void *stream) {
    if (polls == 0 || polls > 100000u) {
        return CUBK_ERR_INVALID_ARG;
    }
    cubk::copy_wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t) stream>>>(polls, status);
    return cubk::check_launch();
}

int cubk_bias_residual_ln_f32(const float *x, const float *bias, const float *residual, const float *gamma,
                              const float *beta, int64_t rows, int channels, float *out, void *stream) {
    return cubk::bias_residual_ln<float>(x, bias, residual, gamma, beta, rows, channels, out,
                                         (cudaStream_t) stream);
}

int cubk_bias_residual_ln_f16(const void *x, const void *bias, const void *residual, const void *gamma,
                              const void *beta, int64_t rows, int channels, void *out, void *stream) {
    return cubk::bias_residual_ln<__half>((const __half *) x, (const __half *) bias, (const __half *) residual,
                                          (const __half *) gamma, (const __half *) beta, rows, channels,
                                          (__half *) out, (cudaStream_t) stream);
}

int cubk_embed_ln_f32(const int32_t *ids, const int8_t *segment_ids, const float *word, const float *pos,
                      const float *type, const float *gamma, const float *beta, int batch, int seq, int hidden,
                      int vocab, int type_vocab, float *out, uint32_t *status, void *stream) {
    return cubk::embed_ln<float>(ids, segment_ids, word, pos, type, gamma, beta, batch, seq, hidden, vocab,
                                 type_vocab, out, status, (cudaStream_t) stream);
}

int cubk_embed_ln_f16(const int32_t *ids, const int8_t *segment_ids, const void *word, const void *pos,
                      const void *type, const void *gamma, const void *beta, int batch, int seq, int hidden,
                      int vocab, int type_vocab, void *out, uint32_t *status, void *stream) {
    return cubk::embed_ln<__half>(ids, segment_ids, (const __half *) word, (const __half *) pos,
                                  (const __half *) type, (const __half *) gamma, (const __half *) beta, batch,
                                  seq, hidden, vocab, type_vocab, (__half *) out, status,
                                  (cudaStream_t) stream);
}

}
