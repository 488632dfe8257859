// Host-side bookkeeping of the C ABI: error text, version, workspace registry.
#include <atomic>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace tidal {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

static std::mutex g_ws_mu;
static std::unordered_map<const void*, WsLayout> g_ws;

const WsLayout* find_ws(const void* d_ws) {
    std::lock_guard<std::mutex> lk(g_ws_mu);
    auto it = g_ws.find(d_ws);
    return it == g_ws.end() ? nullptr : &it->second;   // entries are never moved: node-based map
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_version(void) { return 102; }   // 102: q_src in tidal_rope_append_args, num_pages in tidal_prefill_args,
                                                     //      wait_limit in tidal_exchange_args, reset / status entry points

extern "C" const char* tidal_last_error(void) { return g_err; }

extern "C" uint64_t tidal_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

static int check_geometry(int max_batch, int num_qo_heads, int head_dim, int max_rows, int64_t max_n) {
    TIDAL_REQUIRE(max_batch >= 1 && num_qo_heads >= 1 && head_dim >= 1 && max_rows >= 1 && max_n >= 1, TIDAL_ERR_ARG,
                  "workspace geometry must be positive");
    return TIDAL_OK;
}

extern "C" size_t tidal_ws_bytes(int max_batch, int num_qo_heads, int head_dim, int max_rows, int64_t max_n) {
    if (check_geometry(max_batch, num_qo_heads, head_dim, max_rows, max_n) != TIDAL_OK) return 0;
    return ws_layout(max_batch, num_qo_heads, head_dim, max_rows, max_n).total;
}

extern "C" int tidal_ws_init(void* d_ws, size_t ws_bytes, int max_batch, int num_qo_heads, int head_dim, int max_rows,
                             int64_t max_n, void* stream) {
    TIDAL_REQUIRE(d_ws != nullptr, TIDAL_ERR_ARG, "workspace is NULL");
    TIDAL_REQUIRE(((uintptr_t)d_ws & 255) == 0, TIDAL_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    int rc = check_geometry(max_batch, num_qo_heads, head_dim, max_rows, max_n);
    if (rc != TIDAL_OK) return rc;
    const WsLayout L = ws_layout(max_batch, num_qo_heads, head_dim, max_rows, max_n);
    TIDAL_REQUIRE(ws_bytes >= L.total, TIDAL_ERR_WORKSPACE, "workspace is %zu bytes, geometry needs %zu", ws_bytes, L.total);
    cudaStream_t st = (cudaStream_t)stream;
    // counters that must be zero at rest: status block, histograms, row state
    TIDAL_CUDA_OK(cudaMemsetAsync((char*)d_ws + L.status_off, 0, 256, st));
    TIDAL_CUDA_OK(cudaMemsetAsync((char*)d_ws + L.hist_off, 0, L.cand_off - L.hist_off, st));
    {
        std::lock_guard<std::mutex> lk(g_ws_mu);
        g_ws[d_ws] = L;
    }
    return TIDAL_OK;
}

extern "C" int tidal_ws_release(void* d_ws) {
    std::lock_guard<std::mutex> lk(g_ws_mu);
    g_ws.erase(d_ws);
    return TIDAL_OK;
}

extern "C" int tidal_ws_status(void* d_ws, size_t ws_bytes, void* stream) {
    const WsLayout* L = find_ws(d_ws);
    TIDAL_REQUIRE(L != nullptr, TIDAL_ERR_WORKSPACE, "workspace %p was not initialised with tidal_ws_init", d_ws);
    TIDAL_REQUIRE(ws_bytes >= L->total, TIDAL_ERR_WORKSPACE, "workspace is %zu bytes, layout needs %zu", ws_bytes, L->total);
    uint32_t v = 0;
    cudaStream_t st = (cudaStream_t)stream;
    TIDAL_CUDA_OK(cudaMemcpyAsync(&v, (char*)d_ws + L->status_off, sizeof(v), cudaMemcpyDeviceToHost, st));
    TIDAL_CUDA_OK(cudaStreamSynchronize(st));
    return (int)(v & 0x7fffffffu);
}
