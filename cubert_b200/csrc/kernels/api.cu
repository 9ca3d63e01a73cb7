// Library-wide pieces of the C ABI: version, the last CUDA error of a failed launch, and the
// process-wide tuning switches.
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace cubk {

static thread_local cudaError_t g_last_error = cudaSuccess;

void set_last_error(cudaError_t err) {
    g_last_error = err;
}

// Switches start from the environment (read once, at the first use of any switch) and can be changed
// afterwards with cubk_set_option; reads on the launch path are relaxed atomic loads.
struct OptionSpec {
    const char *env;
    int fallback, lo, hi;
};

static const OptionSpec kOptionSpecs[CUBK_OPT_COUNT] = {
    {"CUBK_BULK_COPY", -1, -1, 1},          // CUBK_OPT_EMBED_STAGED_ROWS
    {"CUBK_SOFTMAX_MASK_SMEM", 1, 0, 1},    // CUBK_OPT_SOFTMAX_MASK_SMEM
    {"CUBK_EXACT_WIDTH_ROWS", 1, 0, 1},     // CUBK_OPT_EXACT_WIDTH_ROWS
    {"CUBK_EXACT_WIDTH_EMBED", 1, 0, 1},    // CUBK_OPT_EXACT_WIDTH_EMBED
    {"CUBK_ATTENTION_TENSOR_MEMORY", 0, 0, 1},   // CUBK_OPT_ATTENTION_TENSOR_MEMORY
};

static std::atomic<int> g_options[CUBK_OPT_COUNT];
static std::once_flag g_options_once;

static void init_options() {
    for (int i = 0; i < CUBK_OPT_COUNT; ++i) {
        int v = kOptionSpecs[i].fallback;
        const char *text = getenv(kOptionSpecs[i].env);
        if (text != nullptr && text[0] != '\0') {
            char *end = nullptr;
            const long parsed = strtol(text, &end, 10);
            if (end != text && parsed >= kOptionSpecs[i].lo && parsed <= kOptionSpecs[i].hi) {
                v = (int) parsed;
            }
        }
        g_options[i].store(v, std::memory_order_relaxed);
    }
}

int option(int id) {
    std::call_once(g_options_once, init_options);
    return g_options[id].load(std::memory_order_relaxed);
}

}  // namespace cubk

extern "C" {

int cubk_version(void) {
    return 110;  // 1.1.0
}

const char *cubk_last_cuda_error(void) {
    return cudaGetErrorString(cubk::g_last_error);
}

int cubk_set_option(int option, int value) {
    if (option < 0 || option >= CUBK_OPT_COUNT || value < cubk::kOptionSpecs[option].lo ||
        value > cubk::kOptionSpecs[option].hi) {
        return CUBK_ERR_INVALID_ARG;
    }
    std::call_once(cubk::g_options_once, cubk::init_options);
    cubk::g_options[option].store(value, std::memory_order_relaxed);
    return CUBK_OK;
}

int cubk_get_option(int option, int *value) {
    if (option < 0 || option >= CUBK_OPT_COUNT || value == nullptr) {
        return CUBK_ERR_INVALID_ARG;
    }
    *value = cubk::option(option);
    return CUBK_OK;
}

}
