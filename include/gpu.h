// Backend facade for cpp-tensorlib builds that use libtlb200.so: array.h and
// storage.h dispatch through tl::gpu (reference include/gpu.h:18-36).  With
// -DTENSORLIB_CUDA the alias selects this directory's cuda.h; the Metal and WebGPU
// headers are the reference's own and stay inert off their platforms.
#pragma once

#include "cuda.h"
#include "metal.h"
#include "webgpu.h"

namespace tl {

#if defined(TENSORLIB_WEBGPU) && defined(__EMSCRIPTEN__)
namespace gpu = webgpu;
#elif defined(TENSORLIB_CUDA) && !defined(__APPLE__)
namespace gpu = cuda;
#else
namespace gpu = metal;
#endif

inline bool gpu_available() { return gpu::available(); }

}  // namespace tl
