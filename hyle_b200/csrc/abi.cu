// ABI version, result strings and the per-device SM count cache.
#include "common.cuh"

namespace hb {

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 148;
  int count = cached[device];
  if (count == 0) {
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    cached[device] = count;  // benign race: every writer stores the same value
  }
  return count;
}

}  // namespace hb

extern "C" int hyle_b200_abi_version(void) { return HYLE_B200_ABI_VERSION; }

extern "C" const char *hyle_b200_result_string(int result) {
  switch (result) {
    case HYLE_B200_OK: return "ok";
    case HYLE_B200_INVALID_VALUE: return "invalid argument";
    case HYLE_B200_NOT_SUPPORTED: return "shape or alignment not supported by this library";
    case HYLE_B200_IO_ERROR: return "file stream: cannot open the file, the range is not inside it, or a read failed";
    case HYLE_B200_STATIC_SCRATCH_EXCEEDED:
      return "count exceeds HYLE_B200_STATIC_MAX_VALUES, the capacity of the library's static scratch";
    default: return cudaGetErrorString(static_cast<cudaError_t>(result));
  }
}

extern "C" int hyle_b200_workspace_clear(hyle_b200_stream_t stream, void *workspace, uint64_t bytes) {
  if (bytes == 0) return HYLE_B200_OK;
  if (workspace == nullptr) return HYLE_B200_INVALID_VALUE;
  return static_cast<int>(cudaMemsetAsync(workspace, 0, bytes, reinterpret_cast<cudaStream_t>(stream)));
}
