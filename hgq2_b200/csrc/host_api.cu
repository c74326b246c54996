// Host-buffer entry of the standalone quantizer: the caller hands in host arrays, the library
// streams them through the GPU in chunks.  Three streams form a pipeline (host->device copies,
// kernels, device->host copies) over a ring of device staging slots, so the two PCIe directions
// and the kernels overlap.  The device staging memory is supplied by the caller.
#include <cuda_runtime.h>

#include <mutex>

#include "hgq_common.cuh"

namespace {

constexpr int kSlots = 3;
constexpr int kMaxDevices = 64;

struct Pipe {
    bool ready = false;
    cudaStream_t h2d, run, d2h;
    cudaEvent_t in_done[kSlots], run_done[kSlots], out_done[kSlots];
};

Pipe g_pipes[kMaxDevices];
std::mutex g_pipe_mutex;

// bytes of one staging slot for `chunk` elements: x,i,f,g,y,dx,di,df fp32 + k uint8, each padded to 256 B
size_t plane(int64_t chunk, size_t elt) { return ((size_t)chunk * elt + 255) / 256 * 256; }
size_t slot_bytes(int64_t chunk) { return 8 * plane(chunk, 4) + plane(chunk, 1); }

int get_pipe(Pipe **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return HGQ_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    Pipe &p = g_pipes[dev];
    if (!p.ready) {
        if ((e = cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        if ((e = cudaStreamCreateWithFlags(&p.run, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        if ((e = cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        for (int s = 0; s < kSlots; ++s) {
            if ((e = cudaEventCreateWithFlags(&p.in_done[s], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
            if ((e = cudaEventCreateWithFlags(&p.run_done[s], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
            if ((e = cudaEventCreateWithFlags(&p.out_done[s], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
        }
        p.ready = true;
    }
    *out = &p;
    return HGQ_OK;
}

}  // namespace

extern "C" size_t hgq_quantize_host_workspace(int64_t chunk_elems) {
    if (chunk_elems <= 0) return 0;
    return kSlots * slot_bytes(chunk_elems);
}

#define HGQ_CUDA(call)                                  \
    do {                                                \
        cudaError_t e_ = (call);                        \
        if (e_ != cudaSuccess) return (int)e_;          \
    } while (0)

extern "C" int hgq_quantize_fwd_bwd_host(const float *hx, const uint8_t *hk, const float *hi, const float *hf,
                                         const float *hg, float *hy, float *hdx, float *hdi, float *hdf, int64_t n,
                                         int round_mode, int overflow_mode, unsigned flags, void *dev_workspace,
                                         size_t dev_workspace_bytes, int64_t chunk_elems) {
    if (n < 0 || chunk_elems <= 0 || chunk_elems % 4 != 0) return HGQ_ERR_SIZE;
    if (n == 0) return HGQ_OK;
    if (!hx || !hk || !hi || !hf || !hy) return HGQ_ERR_NULL;
    const bool bwd = hg != nullptr;
    if (bwd && (!hdx || !hdf)) return HGQ_ERR_NULL;
    if (dev_workspace == nullptr || dev_workspace_bytes < hgq_quantize_host_workspace(chunk_elems)) return HGQ_ERR_WORKSPACE;
    if (!hgq::aligned(dev_workspace, 256)) return HGQ_ERR_ALIGN;
    Pipe *pp = nullptr;
    if (int e = get_pipe(&pp)) return e;
    Pipe &p = *pp;
    const size_t pf = plane(chunk_elems, 4), pk = plane(chunk_elems, 1), sb = slot_bytes(chunk_elems);
    const int64_t nchunks = (n + chunk_elems - 1) / chunk_elems;
    for (int64_t c = 0; c < nchunks; ++c) {
        const int s = (int)(c % kSlots);
        const int64_t off = c * chunk_elems;
        const int64_t m = (n - off < chunk_elems) ? (n - off) : chunk_elems;
        char *base = (char *)dev_workspace + (size_t)s * sb;
        float *dx_ = (float *)(base), *di_ = (float *)(base + pf), *df_ = (float *)(base + 2 * pf),
              *dg_ = (float *)(base + 3 * pf), *dy = (float *)(base + 4 * pf), *ddx = (float *)(base + 5 * pf),
              *ddi = (float *)(base + 6 * pf), *ddf = (float *)(base + 7 * pf);
        uint8_t *dk_ = (uint8_t *)(base + 8 * pf);
        (void)pk;
        if (c >= kSlots) HGQ_CUDA(cudaStreamWaitEvent(p.h2d, p.out_done[s], 0));  // slot drained
        HGQ_CUDA(cudaMemcpyAsync(dx_, hx + off, m * 4, cudaMemcpyHostToDevice, p.h2d));
        HGQ_CUDA(cudaMemcpyAsync(dk_, hk + off, m, cudaMemcpyHostToDevice, p.h2d));
        HGQ_CUDA(cudaMemcpyAsync(di_, hi + off, m * 4, cudaMemcpyHostToDevice, p.h2d));
        HGQ_CUDA(cudaMemcpyAsync(df_, hf + off, m * 4, cudaMemcpyHostToDevice, p.h2d));
        if (bwd) HGQ_CUDA(cudaMemcpyAsync(dg_, hg + off, m * 4, cudaMemcpyHostToDevice, p.h2d));
        HGQ_CUDA(cudaEventRecord(p.in_done[s], p.h2d));

        HGQ_CUDA(cudaStreamWaitEvent(p.run, p.in_done[s], 0));
        if (int e = hgq_quantize_fwd(dx_, dk_, di_, df_, dy, nullptr, m, m, round_mode, overflow_mode, flags, p.run)) return e;
        if (bwd) {
            if (int e = hgq_quantize_bwd(dg_, dx_, dk_, di_, df_, ddx, hdi ? ddi : nullptr, ddf, m, m, round_mode,
                                         overflow_mode, 0u, nullptr, 0, p.run))
                return e;
        }
        HGQ_CUDA(cudaEventRecord(p.run_done[s], p.run));

        HGQ_CUDA(cudaStreamWaitEvent(p.d2h, p.run_done[s], 0));
        HGQ_CUDA(cudaMemcpyAsync(hy + off, dy, m * 4, cudaMemcpyDeviceToHost, p.d2h));
        if (bwd) {
            HGQ_CUDA(cudaMemcpyAsync(hdx + off, ddx, m * 4, cudaMemcpyDeviceToHost, p.d2h));
            if (hdi) HGQ_CUDA(cudaMemcpyAsync(hdi + off, ddi, m * 4, cudaMemcpyDeviceToHost, p.d2h));
            HGQ_CUDA(cudaMemcpyAsync(hdf + off, ddf, m * 4, cudaMemcpyDeviceToHost, p.d2h));
        }
        HGQ_CUDA(cudaEventRecord(p.out_done[s], p.d2h));
    }
    HGQ_CUDA(cudaStreamSynchronize(p.d2h));
    return HGQ_OK;
}
