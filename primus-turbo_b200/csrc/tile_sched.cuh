// Dynamic tile schedule for persistent kernels: CTAs draw tile numbers from a device counter instead of striding by the
// grid size, so a CTA that gets ahead takes more tiles, all SMs finish together and the tiles in flight at any moment
// stay close together in memory.  (Measured on the dual MX quantizer: 16384 x 8192 bf16 4.67 -> 5.72 TB/s.)
//
// The counters live in a small ring of slots inside the library.  A launch takes the next slot, the kernel's last CTA
// clears it, and an event recorded behind the launch tells the host when the slot may be handed out again; when the
// next slot in the ring is still busy, or the stream is being captured into a graph (a replay could run beside another
// launch holding the same slot), the launch falls back to the static schedule (slot -1).  PT_TILE_SCHED_STATIC=1 forces
// the static schedule; PT_TILE_SCHED_IN_GRAPHS=1 allows counters in captured launches, for programs whose graph replays
// never overlap other work of this library on the device.
//
// Everything here has internal linkage: each translation unit that includes this header owns a private ring.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <mutex>

namespace ptb {

constexpr int kTileSchedSlots = 64;
// [slot][0]: tiles handed out beyond each CTA's first; [slot][1]: CTAs that have finished drawing
static __device__ unsigned int g_tile_sched[kTileSchedSlots][2];

// next tile of this CTA after tile t
__device__ __forceinline__ uint32_t tile_sched_next(int slot, uint32_t t) {
    return slot < 0 ? t + gridDim.x : gridDim.x + atomicAdd(&g_tile_sched[slot][0], 1u);
}
// called once per CTA after its last draw; the last CTA clears the slot for its next user
__device__ __forceinline__ void tile_sched_done(int slot) {
    if (slot >= 0 && atomicAdd(&g_tile_sched[slot][1], 1u) == gridDim.x - 1) {
        g_tile_sched[slot][0] = 0u;
        g_tile_sched[slot][1] = 0u;
        __threadfence();
    }
}

struct TileSchedRing {
    cudaEvent_t ev[kTileSchedSlots] = {};
    bool used[kTileSchedSlots] = {};
    unsigned next = 0;
};

static inline TileSchedRing &tile_sched_ring(int dev) {
    static TileSchedRing rings[64];
    return rings[dev];
}
static inline std::mutex &tile_sched_mutex() {
    static std::mutex m;
    return m;
}

// Slot for a launch on `st`, or -1 for the static schedule.
static inline int tile_sched_acquire(cudaStream_t st) {
    if (getenv("PT_TILE_SCHED_STATIC") != nullptr) return -1;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    if (capturing && getenv("PT_TILE_SCHED_IN_GRAPHS") == nullptr) return -1;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    std::lock_guard<std::mutex> lock(tile_sched_mutex());
    TileSchedRing &r = tile_sched_ring(dev);
    const int slot = (int) (r.next % kTileSchedSlots);
    if (r.used[slot] && !capturing) {
        const cudaError_t q = cudaEventQuery(r.ev[slot]);
        if (q != cudaSuccess) {      // its previous user may still be running
            if (q != cudaErrorNotReady) cudaGetLastError();
            return -1;
        }
    }
    ++r.next;
    return slot;
}

// Marks the end of the launch that holds `slot` (call right after the launch, same stream).
static inline void tile_sched_release(int slot, cudaStream_t st) {
    if (slot < 0) return;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return;                      // captured launches are not tracked (see PT_TILE_SCHED_IN_GRAPHS)
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    std::lock_guard<std::mutex> lock(tile_sched_mutex());
    TileSchedRing &r = tile_sched_ring(dev);
    if (r.ev[slot] == nullptr && cudaEventCreateWithFlags(&r.ev[slot], cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        r.used[slot] = false;
        return;
    }
    if (cudaEventRecord(r.ev[slot], st) == cudaSuccess) r.used[slot] = true;
    else cudaGetLastError();
}

}  // namespace ptb
