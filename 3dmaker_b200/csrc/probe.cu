// Measured ceilings for kernels whose work is scattered 4- to 16-byte accesses to an L2-resident table - the hash-grid
// gathers of the forward and the gradient reductions of the backward.  Copy bandwidth says little about them: what
// bounds them is how many independent sectors per second the L1 / L2 path delivers (gathers) and how many reduction
// requests per second the L2 executes (scatter).  nb_probe_random_access issues exactly such accesses at seeded random
// entries of a caller-provided table and nothing else, so that bench.py can put the field kernels' achieved access
// rates next to what the memory system gives a kernel that does no other work.  No counterpart in the reference.
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

__device__ __forceinline__ uint32_t probe_hash(uint32_t v) {
    uint32_t s = v * 747796405u + 2891336453u;
    uint32_t w = ((s >> ((s >> 28u) + 4u)) ^ s) * 277803737u;
    return (w >> 22u) ^ w;
}

// KIND 0: 4-byte gather (ld.global.nc); 1: 8-byte fp32 pair reduction (red.global.add.v2.f32), the scatter's operation
template <int KIND>
__global__ void __launch_bounds__(256) probe_kernel(void* table, uint32_t entry_mask, int per_thread, uint32_t* sink) {
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t h = probe_hash(tid * 9781u + 17u), acc = 0u;
    for (int i = 0; i < per_thread; i++) {
        h = probe_hash(h + (uint32_t)i);
        const uint32_t e = h & entry_mask;
        if (KIND == 0) {
            uint32_t v;
            asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(reinterpret_cast<uint32_t*>(table) + e));
            acc ^= v;
        } else {
            red_add_v2(reinterpret_cast<float*>(table) + (size_t)e * 2, 1.0f, 2.0f);
        }
    }
    if (KIND == 0 && acc == 0x9e3779b9u && sink != nullptr) *sink = acc;   // keeps the loads alive
}

}  // namespace nb

using namespace nb;

// kind 0: gathers of 4 bytes from 2^entries_log2 4-byte entries; kind 1: reductions of 8 bytes into 2^entries_log2
// 8-byte entries.  operations = blocks x 256 threads x per_thread; d_table must hold the entries (kind 1 adds to them).
extern "C" int nb_probe_random_access(int kind, int entries_log2, int blocks, int per_thread, void* d_table, void* stream) {
    if (!d_table || entries_log2 < 4 || entries_log2 > 31 || blocks < 1 || per_thread < 1 || kind < 0 || kind > 1)
        return nb_set_error(NB_ERR_INVALID, "nb_probe_random_access: bad arguments");
    const uint32_t mask = (1u << entries_log2) - 1u;
    if (kind == 0) probe_kernel<0><<<blocks, 256, 0, (cudaStream_t)stream>>>(d_table, mask, per_thread, nullptr);
    else probe_kernel<1><<<blocks, 256, 0, (cudaStream_t)stream>>>(d_table, mask, per_thread, nullptr);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
