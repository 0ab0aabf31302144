// Access to the driver's tensor-map encoder (cuTensorMapEncodeTiled) without linking libcuda: the entry point is
// looked up through the runtime once per process.  Host side only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace b200q {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// nullptr when the driver does not offer the entry point
EncodeTiledFn encode_tiled();
inline bool tma_available() { return encode_tiled() != nullptr; }

}  // namespace b200q
