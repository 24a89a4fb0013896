// rdl_attention_decode_static: decode attention with scratch in a fixed device array (see no_alloc.h).
#include "no_alloc.h"

#include "common.cuh"

// Run counters and partial results of rdl_attention_decode_static.  One copy per device that loads
// the library.  In host code this name is only a handle for cudaGetSymbolAddress, not a device
// address; kernels get the address looked up below.
static __device__ __align__(256) unsigned char g_static_scratch[RDL_STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
void* g_scratch_address[MAX_DEVICES];   // device address of g_static_scratch, per device; null until looked up
}  // namespace

extern "C" int rdl_attention_decode_static(const AttentionArgs* a, void* stream) {
    RDL_REQUIRE(a, "attention_decode_static: missing arguments");
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_heads > 0 && a->n_kv_heads > 0 && a->head_dim > 0 && a->max_splits > 0,
                "attention_decode_static: bad sizes");
    const long long need = rdl_attention_decode_scratch_bytes(a->n_tokens, a->n_heads, a->n_kv_heads, a->head_dim, a->max_splits);
    RDL_REQUIRE(need <= RDL_STATIC_SCRATCH_BYTES,
                "attention_decode_static: this call needs %lld bytes of scratch, the fixed array holds %lld "
                "(fewer tokens, fewer runs, or rdl_attention_decode with scratch of the caller's)",
                need, (long long)RDL_STATIC_SCRATCH_BYTES);
    int device = -1;
    RDL_CUDA(cudaGetDevice(&device), "attention_decode_static");
    RDL_REQUIRE(device >= 0 && device < MAX_DEVICES, "attention_decode_static: device %d is outside the table of %d", device, MAX_DEVICES);
    if (!g_scratch_address[device]) {
        // set-up, once per device, with that device current
        void* p = nullptr;
        RDL_CUDA(cudaGetSymbolAddress(&p, g_static_scratch), "attention_decode_static: address of the scratch array");
        RDL_REQUIRE(p, "attention_decode_static: the scratch array has no device address");
        g_scratch_address[device] = p;
    }
    AttentionArgs b = *a;
    b.scratch = g_scratch_address[device];
    b.scratch_bytes = RDL_STATIC_SCRATCH_BYTES;
    b.counter_bytes = rdl_attention_decode_counter_bytes(a->n_tokens, a->n_kv_heads);
    // the array keeps the last call's contents: the counters must start at zero
    RDL_CUDA(cudaMemsetAsync(b.scratch, 0, (size_t)b.counter_bytes, (cudaStream_t)stream), "attention_decode_static: clearing the counters");
    return rdl_attention_decode(&b, stream);
}
