// Decode attention for callers that cannot allocate device memory.
//
// fpkv_decode_attn needs a scratch buffer from its caller.  Some callers have none to give and no way
// to get one: a serving engine that sized its page pool to take every free byte of HBM at start-up has
// nothing left for a later cudaMalloc; a latency-bound decode loop cannot afford cudaMalloc at all,
// because it synchronises the whole device; and a host that embeds this library under its own memory
// manager may simply forbid allocation in plugin code.  For them the scratch lives here, inside the
// library image, as a fixed array in device memory.
//
// The array belongs to the loaded library, not to a call: every GPU that loads libfpkv.so carries its
// FPKV_STATIC_SCRATCH_BYTES until the process exits, every call on that GPU uses the same bytes, and
// they keep whatever the previous call left.  The words that must start at zero are cleared at the
// head of every call.  Two calls that run on the same GPU at the same time (different streams, or a
// graph replayed next to a live call) would share the bytes and race; run them one after the other.

#include <mutex>

#include "common.cuh"

namespace {

// The scratch itself.  256-byte alignment covers every access the kernels make (16-byte vectors).
static __device__ __align__(256) unsigned char g_static_scratch[FPKV_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_on_device[kMaxDevices] = {};           // device address of the array, per GPU

// In host code `g_static_scratch` is only a handle the runtime uses to find the array; it is not an
// address a kernel could use.  The real device address is looked up once per GPU, with that GPU
// current, and remembered.
int static_scratch_address(void** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FPKV_EARCH;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_on_device[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return FPKV_ELAUNCH;
        g_scratch_on_device[dev] = p;
    }
    *out = g_scratch_on_device[dev];
    return FPKV_OK;
}

}  // namespace

extern "C" int fpkv_decode_attn_static(const fpkv_pool* pool, int32_t layer, void* out, float* lse, const void* q,
                                       int64_t q_stride_b, int64_t q_stride_h, const int64_t* batch_idx,
                                       const void* input_pos, int32_t pos_type, int32_t B, int32_t n_q_heads,
                                       float sm_scale, int32_t* status, void* stream)
{
    if (pool == nullptr || n_q_heads <= 0 || pool->n_heads <= 0) return FPKV_EINVAL;
    if (n_q_heads % pool->n_heads) return FPKV_ESHAPE;
    // What the TMA kernel needs for this head layout does not depend on B or on the context lengths.
    const size_t need = fpkv::decode_tma_workspace_bytes(n_q_heads, pool->n_heads, pool->head_dim);
    if (need > (size_t)FPKV_STATIC_SCRATCH_BYTES) return FPKV_ESTATIC;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != FPKV_OK) return rc;
    // The previous call's leftovers are harmless except for the work counter at the head, which the
    // kernel expects at zero (a call that timed out may have left it dirty): it is cleared on the stream
    // once every argument check has passed, so a refused call enqueues nothing.
    return fpkv::decode_attn_checked(pool, layer, out, lse, q, q_stride_b, q_stride_h, batch_idx, input_pos, pos_type, B,
                                     n_q_heads, sm_scale, scratch, (size_t)FPKV_STATIC_SCRATCH_BYTES, FPKV_DECODE_TMA,
                                     nullptr, status, stream, /*clear_counters=*/true);
}
