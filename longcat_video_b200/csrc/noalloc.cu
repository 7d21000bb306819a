// Block-select for callers that cannot provide a workspace: the scratch lives inside the library.
//
// Some hosts of this library are not allowed to allocate device memory at the point where they
// call it: code running under a memory pool that has been frozen, a plugin that is only handed input
// and output buffers by its runtime, a section of a program that must not touch the CUDA allocator
// because an allocation may synchronise the device.  lcbsa_block_select needs a workspace (the pooled
// Q and K rows) from its caller; lcbsa_block_select_static takes none.  Its workspace is the
// file-scope device array below: kStaticScratchBytes of global memory that every GPU on which this
// library is loaded keeps reserved until the process exits.
//
// There is one array per device and every call on that device uses it, so
//   * two calls whose kernels can overlap on the GPU (different streams, no ordering between them)
//     race on the scratch and must be serialised by the caller;
//   * the array still holds the data of the previous call when the next one starts; nothing in it has
//     to be cleared, because each call overwrites every byte it later reads (the pool kernel fills
//     exactly the rows that the score kernel consumes, the score kernel every key that the top-k
//     kernel reads).
//
// Which kernels run depends on what fits in the array, exactly as for a caller-provided workspace of
// that size.  Pooled rows and 16-bit score keys both fit (16-bit inputs, head_dim 64 or 128;
// lcbsa_select_workspace_bytes_fast <= 32 MiB): pool_kernel, score_gemm_kernel, topk_rows_kernel,
// with the keys in the array behind the pooled rows.  Only the pooled rows fit (a 720p layer with 32
// heads: 23.6 MB of pooled rows, 135 MB of keys), or fp32 inputs: pool_kernel and the fused
// score_topk_kernel, whose scores never leave shared memory.
//
// Inside host code the name of a __device__ array is only a handle, not a device address, so the
// address is resolved with cudaGetSymbolAddress -- once per device, with that device current, by the
// first call made on that device.  That first call should therefore be made outside any stream
// capture; later calls only launch kernels.
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB: pooled Q + K of a 720p layer (32 heads) is 23.6 MB
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_select_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
unsigned char* g_scratch_ptr[kMaxDevices] = {};  // resolved device address of the array, per device

// Device address of the scratch array on the current device (resolved on first use).
unsigned char* scratch_on_current_device(cudaError_t* err) {
    int dev = -1;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= kMaxDevices) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_select_scratch);
        if (*err != cudaSuccess) return nullptr;
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    return g_scratch_ptr[dev];
}

}  // namespace

extern "C" {

size_t lcbsa_static_scratch_bytes(void) { return kStaticScratchBytes; }

int lcbsa_block_select_static(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk, int nsel,
                              int cap, int32_t* idx, int32_t* cnt, void* stream) {
    char msg[256];
    if (q && k)  // a malformed descriptor is an argument error, not a workspace error
        for (int i = 0; i < 4; ++i)
            if (q->size[i] < 0 || k->size[i] < 0) {
                lcbsa::set_last_error("block_select_static: negative size in a tensor description");
                return LCBSA_EINVAL;
            }
    const size_t need = lcbsa_select_workspace_bytes(q, k, gq, gk);
    if (need == 0) {
        lcbsa::set_last_error("block_select_static: bad tensor or grid description");
        return LCBSA_EINVAL;
    }
    if (need > kStaticScratchBytes) {
        snprintf(msg, sizeof(msg),
                 "block_select_static: this problem needs %zu bytes of scratch, the built-in array holds %zu; "
                 "use lcbsa_block_select with a caller-provided workspace",
                 need, kStaticScratchBytes);
        lcbsa::set_last_error(msg);
        return LCBSA_EWORKSPACE;
    }
    cudaError_t e = cudaSuccess;
    unsigned char* scratch = scratch_on_current_device(&e);
    if (scratch == nullptr) {
        snprintf(msg, sizeof(msg), "block_select_static: cannot resolve the scratch array: %s", cudaGetErrorString(e));
        lcbsa::set_last_error(msg);
        return LCBSA_ECUDA;
    }
    // From here on this is the ordinary path on a workspace of kStaticScratchBytes: lcbsa_block_select picks the
    // three-kernel form when the score keys fit behind the pooled rows and the two-kernel form otherwise; no allocation.
    return lcbsa_block_select(q, k, gq, gk, nsel, cap, idx, cnt, scratch, kStaticScratchBytes, stream);
}

}  // extern "C"
