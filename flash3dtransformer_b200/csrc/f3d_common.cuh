// Shared host/device helpers for the Flash3D B200 kernels: status codes, the thread-local error
// string behind f3d_last_error(), launch checking, and the per-device scratch workspace.
//
// Error convention: the reference logs a CUDA error and calls exit() (src/common/runtime.h:29-34) and
// throws std::runtime_error for argument errors (src/common/runtime.h:36-86).  This library never
// exits: every entry point returns 0 or a negative status and leaves a message for f3d_last_error().
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#define F3D_OK 0
#define F3D_ERR_ARG (-1)      // bad shape / enum / size (reference: throw_format_error)
#define F3D_ERR_CUDA (-2)     // CUDA runtime error (reference: exit())
#define F3D_ERR_UNSUPPORTED (-3)
#define F3D_ERR_DEVICE_STATUS (-4)  // a kernel reported a bounded wait running out

namespace f3d {

char *err_buf();                       // thread-local, 512 bytes
int set_error(int code, const char *fmt, ...);

// Grow-only scratch workspace, one block per (device, slot, stream).  The returned pointer stays valid until a later
// call with the same key asks for more bytes.  All kernels of one entry point run on the caller's stream, so reuse
// across calls on that stream is ordered; calls on different streams get different blocks and may overlap on the GPU.
// When a block has to grow, only its own stream is waited for before the old block is freed.  What stays with the
// caller, as with any CUDA stream: two host threads must not issue calls on the SAME stream at the same time.
int workspace(int device, int slot, size_t bytes, cudaStream_t stream, void **out);
void workspace_release_all();

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device), for any device ordinal and from any
// host thread.
int ensure_dynamic_smem(const void *kernel, int device, int bytes);
int sm_count(int device);              // multiprocessors of a device (cached)

bool sync_flag();
void count_launches(int n);            // kernels launched by this library since load (f3d_launch_count)

static inline int check_launch(const char *what, int kernels = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(F3D_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  count_launches(kernels);
  return F3D_OK;
}

static inline int maybe_sync(cudaStream_t s, const char *what) {
  if (!sync_flag()) return F3D_OK;
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return set_error(F3D_ERR_CUDA, "%s (sync): %s", what, cudaGetErrorString(e));
  return F3D_OK;
}

#define F3D_CUDA_TRY(expr)                                                                  \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) return f3d::set_error(F3D_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define F3D_TRY(expr)            \
  do {                           \
    int _s = (expr);             \
    if (_s != F3D_OK) return _s; \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  explicit DeviceGuard(int dev) {
    // A host thread that has made no runtime call yet (an autograd worker whose first operator is one of ours) has no
    // context bound, and driver entry points such as cuTensorMapEncodeTiled then fail with "invalid context":
    // cudaSetDevice binds the device's primary context, so it runs once per thread even when the device is unchanged.
    static thread_local int bound = -1;
    cudaGetDevice(&prev);
    if (prev != dev || bound != dev) {
      cudaSetDevice(dev);
      bound = dev;
      changed = prev != dev;
    }
  }
  ~DeviceGuard() { if (changed) cudaSetDevice(prev); }
};

static inline uint32_t cdiv_u32(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

// feature element types accepted by the pooling / unpooling entry points
enum FeatDtype { F3D_BF16 = 0, F3D_FP16 = 1, F3D_FP32 = 2 };

}  // namespace f3d
