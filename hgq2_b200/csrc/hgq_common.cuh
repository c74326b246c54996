// Host-side helpers shared by the translation units of the library: status codes, argument
// checks, launch accounting and the launch geometry of the broadcast-layout kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/hgq_b200.h"

namespace hgq {

constexpr int kThreads = 256;       // CTA size of every streaming kernel
constexpr int64_t kMaxParamAbs = 100;
enum : int { ACT_NONE = 0, ACT_RELU = 1 };  // fused output activations of the contraction kernels

extern std::atomic<int64_t> g_launches;

// Number of SMs of the current device (148 on a B200: 2 dies x 74), asked of the runtime once per device.  Grid sizes and
// the workspace sizes that follow from them both come from here, so they agree on whatever part the library runs on.
inline int num_sms() {
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return 148;  // no device in this process (host-only use of the size queries)
    }
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
            cudaGetLastError();
            v = 148;
        }
        cache[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

inline int check_launch() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();  // clear the non-sticky error so the next call starts clean
        return (int)e;
    }
    return HGQ_OK;
}

// 256-bit global accesses (sm_100): one instruction moves a whole 32-byte sector per thread.  Two 128-bit accesses to the
// two halves of a sector are two requests for that sector wherever the first level cache does not merge them (streaming
// stores, cache-bypassing loads), and the rate of sector requests between an SM and L2 is what bounds several of the
// kernels here well before HBM does.  Addresses must be 32-byte aligned.
#ifdef __CUDACC__
__device__ __forceinline__ void ldg8(const float *p, float (&v)[8]) {  // read-only data, kept in L1 like __ldg
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(p));
}
__device__ __forceinline__ void ldcs8(const float *p, float (&v)[8]) {  // streaming: read once
    asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(p));
}
__device__ __forceinline__ void stcs8(float *p, const float (&v)[8]) {  // streaming store of a whole sector
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
                 "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                 : "memory");
}
#endif

__host__ __device__ inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Division of a non-negative 31-bit number by an invariant divisor through one 64-bit multiply: n / d == (n * mul) >> shift
// for every 0 <= n < 2^31 with shift = 31 + ceil(log2 d), mul = ceil(2^shift / d).
struct FastDiv {
    uint64_t mul;
    int shift;
    uint32_t d;
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    int l = 0;
    while ((1u << l) < d) ++l;
    f.shift = 31 + l;
    f.mul = ((((uint64_t)1) << f.shift) + d - 1) / d;
    f.d = d;
    return f;
}
__host__ __device__ inline uint32_t fastdiv(uint32_t n, const FastDiv &f) { return (uint32_t)(((uint64_t)n * f.mul) >> f.shift); }

inline int pow2ceil(int64_t v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

// Geometry of a broadcast-layout launch: x is [rows, P], parameters are [P].  A CTA is a
// TX x TY arrangement of 256 threads; a thread owns VEC consecutive columns for the whole launch
// (so the parameters live in registers and column reductions need no atomics) and walks rows
// r0+ty, r0+ty+TY, ...  grid = (colTiles, rowBlocks).
struct BcastGeom {
    int vec;            // 4 (128-bit accesses) or 1
    int64_t V;          // P / vec: vector columns
    int TX, TY;         // TX * TY == kThreads, TX a power of two
    int64_t colTiles;   // ceil(V / TX)
    int rowBlocks;      // grid.y
    int64_t rowsPerBlock;
};

inline BcastGeom bcast_geom(int64_t rows, int64_t P, bool can_vec, int unroll) {
    BcastGeom g;
    g.vec = (can_vec && P % 4 == 0) ? 4 : 1;
    g.V = P / g.vec;
    g.TX = (int)(g.V >= kThreads ? kThreads : pow2ceil(g.V));
    g.TY = kThreads / g.TX;
    g.colTiles = (g.V + g.TX - 1) / g.TX;
    const int64_t target = (int64_t)num_sms() * 8;
    int64_t rb = (target + g.colTiles - 1) / g.colTiles;
    const int64_t maxrb = (rows + (int64_t)g.TY * unroll - 1) / ((int64_t)g.TY * unroll);
    if (rb > maxrb) rb = maxrb;
    if (rb < 1) rb = 1;
    if (rb > 65535) rb = 65535;
    g.rowsPerBlock = (rows + rb - 1) / rb;
    g.rowBlocks = (int)((rows + g.rowsPerBlock - 1) / g.rowsPerBlock);
    return g;
}

}  // namespace hgq
