// Library-wide host state: last-error text, per-device status word, SM count.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace llmb {

static thread_local char g_last_error[512] = "";

void set_last_error(const char *msg) {
    std::snprintf(g_last_error, sizeof(g_last_error), "%s", msg);
}

int cuda_fail(cudaError_t e, const char *file, int line) {
    const char *base = std::strrchr(file, '/');
    std::snprintf(g_last_error, sizeof(g_last_error), "CUDA error %d (%s) at %s:%d", (int)e, cudaGetErrorString(e),
                  base ? base + 1 : file, line);
    return LLMB_ERR_CUDA;
}

static std::mutex g_mu;
static __device__ __align__(256) int g_status_word[64];  // [0] is the status word; the rest pads the line
static int *g_status[64] = {};
static int g_sms[64] = {};

int *device_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_status[dev]) {
        // a variable of the module, not an allocation: every device that loads the library has its own copy,
        // zero when the module is loaded, and looking up its address allocates nothing
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        g_status[dev] = static_cast<int *>(p);
    }
    return g_status[dev];
}

int sm_count_cached() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

}  // namespace llmb

extern "C" const char *llmb_last_error(void) { return llmb::g_last_error; }

extern "C" int llmb_device_status(int *status_out) {
    int *p = llmb::device_status_ptr();
    if (!p || !status_out) return LLMB_ERR_INVALID;
    LLMB_CUDA_OK(cudaDeviceSynchronize());
    LLMB_CUDA_OK(cudaMemcpy(status_out, p, sizeof(int), cudaMemcpyDeviceToHost));
    LLMB_CUDA_OK(cudaMemset(p, 0, sizeof(int)));
    return LLMB_OK;
}

extern "C" const char *llmb_build_info(void) {
    return "llm_b200 sm_100a: gemv_f16(bulk-copy pipeline) attn_decode(split-kv) embed_rope argmax bf16_to_fp16";
}
