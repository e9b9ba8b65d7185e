// Which SMs sit on which die of the B200?
//
// A B200 is two dies, each with its own half of the L2; an SM reaches the other die's L2 across the die-to-die
// link, at a higher latency.  The tensor-core GEMM uses this to keep the A panel of a rasterisation group on one
// die (see tc_gemm_kernel, "die-aware walk"): it needs a table smid -> die.  The numbering of the SMs is not
// documented and differs from chip to chip (different SMs are fused off), so the table is measured once per
// process: one CTA per SM times a chain of dependent L2 hits to ONE address; the SMs split into a near group
// (about 250 cycles) and a far group (about 320).  If the split is not clean — another GPU generation, a busy GPU —
// the table is not produced and the GEMM keeps its die-oblivious walk.

#include "pg_internal.h"

#include <stdlib.h>
#include <string.h>

namespace pgb {

constexpr int TOPO_CHAIN = 96;      // dependent loads per measurement
constexpr int TOPO_REPS = 3;        // the fastest of these is kept

__global__ void topology_probe_kernel(const unsigned *cell, unsigned *out_smid, unsigned *out_cycles) {
    extern __shared__ unsigned char topo_pad[];      // sized by the launch so that one CTA fills an SM
    if (threadIdx.x != 0) return;
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    unsigned v = 0, best = 0xFFFFFFFFu;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(cell) : "memory");          // bring the line into L2
    for (int rep = 0; rep < TOPO_REPS; ++rep) {
        long long t0, t1;
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(t0) :: "memory");
        // each address needs the previous value (the cell holds zero): the loads run one after the other
        for (int i = 0; i < TOPO_CHAIN; ++i)
            asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(cell + v) : "memory");
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(t1) :: "memory");
        const unsigned c = (unsigned)((t1 - t0) / TOPO_CHAIN) + (v & 1u);
        best = c < best ? c : best;
    }
    out_smid[blockIdx.x] = smid;
    out_cycles[blockIdx.x] = best;
}

// Fills table[smid] (0 / 1) for smid < 256 on the current device.  Returns true when the SMs fall into two clean
// groups of comparable size; `scratch` is a device buffer of at least 4 KB that the caller owns.
bool measure_die_table(unsigned char table[256], void *scratch, cudaStream_t stream) {
    const int sms = device_sm_count();
    if (sms < 2 || sms > 256 || !scratch) return false;
    unsigned *cell = (unsigned *)scratch;                 // 256 bytes, zero
    unsigned *d_smid = cell + 64, *d_cyc = d_smid + 256;  // 2 x 1 KB
    if (cudaMemsetAsync(scratch, 0, 4096, stream) != cudaSuccess) { cudaGetLastError(); return false; }
    int max_smem = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const int smem = max_smem > 0 ? max_smem - 1024 : 0;          // more than half an SM's shared memory: one CTA per SM
    if (cudaFuncSetAttribute(topology_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    unsigned h_smid[256], h_cyc[256];
    for (int attempt = 0; attempt < 2; ++attempt) {
        topology_probe_kernel<<<sms, 32, smem, stream>>>(cell, d_smid, d_cyc);
        note_launch();
        if (cudaGetLastError() != cudaSuccess) return false;
        if (cudaMemcpyAsync(h_smid, d_smid, sms * 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
            cudaMemcpyAsync(h_cyc, d_cyc, sms * 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
            cudaStreamSynchronize(stream) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
    }
    unsigned lo = 0xFFFFFFFFu, hi = 0;
    bool seen[256] = {false};
    for (int i = 0; i < sms; ++i) {
        if (h_smid[i] >= 256 || seen[h_smid[i]]) return false;   // two CTAs on one SM: the launch did not spread out
        seen[h_smid[i]] = true;
        lo = h_cyc[i] < lo ? h_cyc[i] : lo;
        hi = h_cyc[i] > hi ? h_cyc[i] : hi;
    }
    if (hi - lo < 30) return false;                               // one group: no second die to tell apart
    const unsigned mid = (lo + hi) / 2;
    // clean split: nobody within 10 cycles of the threshold, both groups at least a third of the SMs
    int near = 0;
    memset(table, 0, 256);
    for (int i = 0; i < sms; ++i) {
        const unsigned c = h_cyc[i];
        if ((c > mid ? c - mid : mid - c) < 10) return false;
        if (c < mid) ++near; else table[h_smid[i]] = 1;
    }
    return near * 3 >= sms && (sms - near) * 3 >= sms;
}

}  // namespace pgb
