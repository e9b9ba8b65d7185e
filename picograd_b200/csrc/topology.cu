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

constexpr int TOPO_CHAIN = 64;      // dependent loads per measurement
constexpr int TOPO_REPS = 2;        // the faster of these is kept
constexpr int TOPO_ADDRS = 24;      // addresses probed; their lines are spread over the L2 slices of both dies
constexpr size_t TOPO_STRIDE = (1u << 20) + 256;     // bytes between probed addresses

__global__ void topology_probe_kernel(const unsigned *cells, unsigned *out_smid, unsigned *out_cycles) {
    extern __shared__ unsigned char topo_pad[];      // sized by the launch so that one CTA fills an SM
    if (threadIdx.x != 0) return;
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    out_smid[blockIdx.x] = smid;
    for (int a = 0; a < TOPO_ADDRS; ++a) {
        const unsigned *cell = cells + (size_t)a * (TOPO_STRIDE / 4);
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
        out_cycles[blockIdx.x * TOPO_ADDRS + a] = best;
    }
}

// Fills table[smid] (0 / 1) for smid < 256 on the current device; true when the SMs fall into two clean groups of
// comparable size.  A line lives in the L2 of one die: for each probed address the SMs of that die see a latency
// below the median over all SMs, the others above, so two SMs of one die agree on (nearly) every address and two SMs
// of different dies disagree on (nearly) every one.  Each SM is compared with the first one measured.
bool measure_die_table(unsigned char table[256], cudaStream_t stream) {
    const int sms = device_sm_count();
    if (sms < 2 || sms > 256) { set_error("die topology: %d SMs", sms); return false; }
    const size_t cells_bytes = (size_t)TOPO_ADDRS * TOPO_STRIDE, out_bytes = 256 * 4 + 256 * TOPO_ADDRS * 4;
    char *buf = nullptr;
    if (cudaMalloc((void **)&buf, cells_bytes + out_bytes) != cudaSuccess) { cudaGetLastError(); return false; }
    struct Free { char *p; ~Free() { cudaFree(p); } } guard{buf};
    unsigned *cells = (unsigned *)buf, *d_smid = (unsigned *)(buf + cells_bytes), *d_cyc = d_smid + 256;
    if (cudaMemsetAsync(buf, 0, cells_bytes + out_bytes, stream) != cudaSuccess) { cudaGetLastError(); return false; }
    int max_smem = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const int smem = max_smem > 0 ? max_smem - 1024 : 0;          // more than half an SM's shared memory: one CTA per SM
    if (cudaFuncSetAttribute(topology_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    static unsigned h_smid[256], h_cyc[256 * TOPO_ADDRS];
    topology_probe_kernel<<<sms, 32, smem, stream>>>(cells, d_smid, d_cyc);
    note_launch();
    if (cudaGetLastError() != cudaSuccess ||
        cudaMemcpyAsync(h_smid, d_smid, sms * 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaMemcpyAsync(h_cyc, d_cyc, (size_t)sms * TOPO_ADDRS * 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    bool seen[256] = {false};
    for (int i = 0; i < sms; ++i) {
        if (h_smid[i] >= 256 || seen[h_smid[i]]) {               // two CTAs on one SM: the launch did not spread out
            set_error("die topology: SM %u measured twice", h_smid[i]);
            return false;
        }
        seen[h_smid[i]] = true;
    }
    // per address: the median over the SMs, and whether the address separates them at all
    unsigned median[TOPO_ADDRS];
    bool useful[TOPO_ADDRS];
    int n_useful = 0;
    for (int a = 0; a < TOPO_ADDRS; ++a) {
        unsigned col[256];
        for (int i = 0; i < sms; ++i) col[i] = h_cyc[i * TOPO_ADDRS + a];
        for (int i = 1; i < sms; ++i) {                          // insertion sort: 148 values
            const unsigned x = col[i];
            int j = i - 1;
            while (j >= 0 && col[j] > x) { col[j + 1] = col[j]; --j; }
            col[j + 1] = x;
        }
        median[a] = (col[sms / 2 - 1] + col[sms / 2]) / 2;
        useful[a] = col[sms - sms / 8] - col[sms / 8] >= 30;      // the two groups are >= 30 cycles apart
        n_useful += useful[a] ? 1 : 0;
    }
    if (n_useful < TOPO_ADDRS / 2) {
        set_error("die topology: only %d of %d probed addresses separate the SMs into two latency groups", n_useful, TOPO_ADDRS);
        return false;
    }
    // (any table gives correct products: it only decides which tiles a CTA pair takes.  A few SMs may sit between
    // the groups — they go with the majority of their addresses; many of them mean the picture is not two dies.)
    int group1 = 0, unclear = 0;
    memset(table, 0, 256);
    for (int i = 0; i < sms; ++i) {
        int agree = 0;
        for (int a = 0; a < TOPO_ADDRS; ++a)
            if (useful[a] && ((h_cyc[i * TOPO_ADDRS + a] < median[a]) == (h_cyc[a] < median[a]))) ++agree;
        if (agree * 4 > n_useful && agree * 4 < n_useful * 3) ++unclear;   // neither with the first SM nor against it
        if (agree * 2 < n_useful) { table[h_smid[i]] = 1; ++group1; }
    }
    if (unclear * 8 > sms) {
        set_error("die topology: %d of %d SMs sit between the two latency groups", unclear, sms);
        return false;
    }
    if (group1 * 3 < sms || (sms - group1) * 3 < sms) {
        set_error("die topology: groups of %d and %d SMs", sms - group1, group1);
        return false;
    }
    return true;
}

}  // namespace pgb
