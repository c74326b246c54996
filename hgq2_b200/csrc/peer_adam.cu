// Gradient exchange over NVLink peer memory fused with the optimizer update: the data-parallel tail of a QAT step on one
// node (one process per GPU) as ONE kernel per rank instead of an NCCL all-reduce followed by the Adam kernel.
//
// The reference leaves this to Keras' distribution strategy plus optimizer.apply (nothing in the HGQ2 tree); the math of
// the update is hgq_adam_step's (optim.cu): Keras Adam with the MonoL1 regulariser and the variable constraints folded in.
//
// Every rank owns an exchange buffer that its peers have mapped (CUDA IPC):
//     [2 slots][n_pad floats]  its gradient bucket of step t in slot t & 1
//     [2 slots][chunks] uint64 per chunk of kPaChunk floats: the step number once the chunk of that slot is complete
// CTA c of the kernel (the same grid on every rank)
//   1. copies chunk c of its own gradients into its own slot, fences, and publishes the step number in the chunk's flag;
//   2. waits -- a bounded number of polls with a sleep between them -- until the same flag of every peer shows the step number
//      (plain peer loads over NVLink: no switch-side reduction, no collective library);
//   3. adds the chunk over the ranks in rank order (the same order on every rank, so all ranks compute bit-identical sums
//      and their parameters never drift apart) and applies the update to its own copy of the parameters.
// Two slots are enough: a rank can only write slot t & 1 again at step t + 2, after it has seen every peer's flag of step
// t + 1, which a peer publishes after it has finished reading step t.
// CTAs of one GPU never wait for one another, only for the CTA of the same index on the other GPUs, which has published
// before it waits: no launch-order assumption within a GPU.  A wait that runs out sets bit 1 of the status word and the
// CTA returns without touching the parameters; the host sees the word behind the step.
#include <cuda_runtime.h>

#include <cstring>

#include "hgq_common.cuh"

namespace hgq {

constexpr int kPaChunk = 2048;           // floats per CTA: 256 threads x 2 float4
constexpr unsigned kPaStatusBit = 2u;
constexpr int kPaMaxWorld = 16;

struct PaPeers {
    float *buf[kPaMaxWorld];
};

__device__ __forceinline__ void pa_store_release(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long pa_load_acquire(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 pa_load4(const float *p) {  // re-fetched on every access: never a stale cached line
    return __ldcv(reinterpret_cast<const float4 *>(p));
}

__global__ void __launch_bounds__(kThreads) k_adam_peers(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ m,
                                                         float *__restrict__ v, const float *__restrict__ lo,
                                                         const float *__restrict__ hi, const float *__restrict__ l1, int64_t n,
                                                         int64_t n_pad, int chunks, float lr, float b1, float b2, float eps,
                                                         const long long *__restrict__ step, PaPeers peers, int world, int rank,
                                                         unsigned max_polls, unsigned *status) {
    const long long t = *step + 1;
    const int slot = (int)(t & 1);
    const int c = blockIdx.x, tid = threadIdx.x;
    const int64_t e0 = (int64_t)c * kPaChunk;
    float *mine = peers.buf[rank] + (int64_t)slot * n_pad;
    // 1. publish this chunk of the local gradients (the tail past n is zero-filled so that float4 accesses stay in range)
#pragma unroll
    for (int j = 0; j < kPaChunk / (kThreads * 4); ++j) {
        const int64_t e = e0 + (int64_t)(j * kThreads + tid) * 4;
        if (e < n_pad) {
            float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e + 3 < n) q = *reinterpret_cast<const float4 *>(g + e);
            else {
                if (e < n) q.x = g[e];
                if (e + 1 < n) q.y = g[e + 1];
                if (e + 2 < n) q.z = g[e + 2];
            }
            *reinterpret_cast<float4 *>(mine + e) = q;
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence_system();
        unsigned long long *flags = reinterpret_cast<unsigned long long *>(peers.buf[rank] + 2 * n_pad) + (int64_t)slot * chunks;
        pa_store_release(flags + c, (unsigned long long)t);
    }
    // 2. wait for the same chunk of every peer (thread r polls rank r)
    bool ok = true;
    if (tid < world && tid != rank) {
        const unsigned long long *flag =
            reinterpret_cast<const unsigned long long *>(peers.buf[tid] + 2 * n_pad) + (int64_t)slot * chunks + c;
        ok = false;
        for (unsigned it = 0; it < max_polls; ++it) {
            if (pa_load_acquire(flag) == (unsigned long long)t) { ok = true; break; }
            if (it > 64) __nanosleep(200);  // a peer that is far behind: stop hammering the link
        }
    }
    if (!__syncthreads_and(ok ? 1 : 0)) {
        if (tid == 0 && status) atomicOr(status, kPaStatusBit);
        return;
    }
    // 3. sum over the ranks in rank order, then the update
    const float c1 = 1.f - powf(b1, (float)t);
    const float c2 = 1.f - powf(b2, (float)t);
    const float alpha = lr * sqrtf(c2) / c1;
    const float scale = 1.f / (float)world;
#pragma unroll
    for (int j = 0; j < kPaChunk / (kThreads * 4); ++j) {
        const int64_t e = e0 + (int64_t)(j * kThreads + tid) * 4;
        if (e >= n) continue;
        // every rank's piece is requested before the first one is used: one NVLink round trip for all of them, not one each
        float4 q[kPaMaxWorld];
#pragma unroll
        for (int r = 0; r < kPaMaxWorld; ++r)
            if (r < world) q[r] = pa_load4(peers.buf[r] + (int64_t)slot * n_pad + e);
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kPaMaxWorld; ++r)
            if (r < world) { s.x += q[r].x; s.y += q[r].y; s.z += q[r].z; s.w += q[r].w; }
        const float sv[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t ee = e + k;
            if (ee >= n) break;
            float ge = sv[k] * scale;
            if (l1) ge += l1[ee];
            const float me = b1 * m[ee] + (1.f - b1) * ge;
            const float ve = b2 * v[ee] + (1.f - b2) * ge * ge;
            float we = w[ee] - alpha * me / (sqrtf(ve) + eps);
            if (lo) we = fmaxf(we, lo[ee]);
            if (hi) we = fminf(we, hi[ee]);
            m[ee] = me;
            v[ee] = ve;
            w[ee] = we;
        }
    }
}

__global__ void k_step_inc_peers(long long *step) { *step += 1; }

static int64_t pa_pad(int64_t n) { return (n + kPaChunk - 1) / kPaChunk * kPaChunk; }

}  // namespace hgq

using namespace hgq;

extern "C" size_t hgq_peer_exchange_bytes(int64_t n) {
    if (n <= 0) return 0;
    const int64_t n_pad = pa_pad(n), chunks = n_pad / kPaChunk;
    return (size_t)(2 * n_pad) * sizeof(float) + (size_t)(2 * chunks) * sizeof(unsigned long long);
}

extern "C" int hgq_peer_buffer_create(size_t bytes, void **dev_ptr, void *ipc_handle_64) {
    if (dev_ptr == nullptr || ipc_handle_64 == nullptr) return HGQ_ERR_NULL;
    if (bytes == 0) return HGQ_ERR_SIZE;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();  // the failure is reported through the return value, not left behind for the next launch check
        return (int)e;
    }
    e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(ipc_handle_64), p);
    if (e != cudaSuccess) {
        cudaFree(p);
        cudaGetLastError();
        return (int)e;
    }
    *dev_ptr = p;
    return HGQ_OK;
}

extern "C" int hgq_peer_buffer_open(const void *ipc_handle_64, void **dev_ptr) {
    if (dev_ptr == nullptr || ipc_handle_64 == nullptr) return HGQ_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle_64, sizeof(h));
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();  // e.g. a peer on another node or without peer access: the caller falls back to NCCL
        return (int)e;
    }
    *dev_ptr = p;
    return HGQ_OK;
}

extern "C" int hgq_peer_buffer_close(void *dev_ptr) {
    if (dev_ptr == nullptr) return HGQ_OK;
    return (int)cudaIpcCloseMemHandle(dev_ptr);
}

extern "C" int hgq_peer_buffer_destroy(void *dev_ptr) {
    if (dev_ptr == nullptr) return HGQ_OK;
    return (int)cudaFree(dev_ptr);
}

extern "C" int hgq_adam_step_peers(float *w, const float *g, float *m, float *v, const float *lo, const float *hi,
                                   const float *l1, int64_t n, float lr, float beta1, float beta2, float eps, long long *step,
                                   void *const *peer_bufs, int world, int rank, unsigned max_polls, unsigned *status,
                                   void *stream) {
    if (n < 0) return HGQ_ERR_SIZE;
    if (n == 0) return HGQ_OK;
    if (!w || !g || !m || !v || !step || !peer_bufs) return HGQ_ERR_NULL;
    if (world < 1 || world > kPaMaxWorld || rank < 0 || rank >= world || max_polls == 0) return HGQ_ERR_SIZE;
    if (!aligned(g, 16)) return HGQ_ERR_ALIGN;
    PaPeers peers{};
    for (int r = 0; r < world; ++r) {
        if (peer_bufs[r] == nullptr) return HGQ_ERR_NULL;
        if (!aligned(peer_bufs[r], 16)) return HGQ_ERR_ALIGN;
        peers.buf[r] = static_cast<float *>(peer_bufs[r]);
    }
    const int64_t n_pad = pa_pad(n);
    const int64_t chunks = n_pad / kPaChunk;
    if (chunks > 65535 * 16) return HGQ_ERR_SIZE;
    cudaStream_t st = (cudaStream_t)stream;
    k_adam_peers<<<(unsigned)chunks, kThreads, 0, st>>>(w, g, m, v, lo, hi, l1, n, n_pad, (int)chunks, lr, beta1, beta2, eps, step,
                                                       peers, world, rank, max_polls, status);
    if (int e = check_launch()) return e;
    k_step_inc_peers<<<1, 1, 0, st>>>(step);
    return check_launch();
}
