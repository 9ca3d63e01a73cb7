// Host-side arithmetic of the key plan (see Bert<T>::KeyPlan): where each sequence's kept keys end and how
// sequences group by that extent. Plain functions on host arrays, so that they can be tested without a GPU.
#pragma once

#include <cstddef>
#include <cstdint>

namespace cubert {

// Key extent of one mask row of `seq` entries: the position after the last non-zero entry, rounded up to a
// multiple of `granule` and capped at `seq`; `seq` when no entry is non-zero (the reference then attends to
// every position uniformly, src/cuBERT/op_att/AttentionMask.cpp:14-16 with AttentionSelf.cpp:58-60).
inline int key_extent(const int8_t *mask_row, int seq, int granule) {
    int last = seq - 1;
    while (last >= 0 && mask_row[last] == 0) {
        --last;
    }
    if (last < 0) {
        return seq;
    }
    const int extent = (last / granule + 1) * granule;
    return extent > seq ? seq : extent;
}

// Counting sort of `batch` sequences by extent (extents are multiples of `granule` or equal to `seq`).
// order[i] = the i-th sequence in order of growing extent (ties in batch order); group g covers
// order[start[g] .. start[g + 1]) and has extent group_extent[g]. Returns the number of groups, or 0 when
// there would be more than `max_groups` distinct extents.
inline int group_by_extent(const int32_t *extents, size_t batch, int seq, int granule, int max_groups, int32_t *order,
                           int *start, int *group_extent) {
    const int buckets = (seq + granule - 1) / granule;
    if (buckets > max_groups) {
        return 0;
    }
    int count[64 + 2] = {};
    int first[64 + 2] = {};
    if (buckets > 64) {
        return 0;
    }
    for (size_t b = 0; b < batch; ++b) {
        count[(extents[b] + granule - 1) / granule] += 1;
    }
    int groups = 0, at = 0;
    for (int k = 1; k <= buckets; ++k) {
        first[k] = at;
        if (count[k] > 0) {
            start[groups] = at;
            group_extent[groups] = k * granule > seq ? seq : k * granule;
            ++groups;
        }
        at += count[k];
    }
    start[groups] = at;
    for (size_t b = 0; b < batch; ++b) {
        order[first[(extents[b] + granule - 1) / granule]++] = (int32_t) b;
    }
    return groups;
}

}  // namespace cubert
