// Host-side support of the tcgen05 kernels: tensor-map encoding and the device status words.
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "tc_common.cuh"

namespace sparta {
namespace tc {

__device__ int32_t g_status[4];

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* map, const void* base, int dtype, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return SPARTA_ERR_DRIVER;
  if (!aligned(base, 16)) return SPARTA_ERR_ALIGN;
  CUtensorMapDataType dt;
  if (dtype == SPARTA_F16) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  else if (dtype == SPARTA_BF16) dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  else if (dtype == kTensorMapU8) dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  else if (dtype == kTensorMapU32) dt = CU_TENSOR_MAP_DATA_TYPE_UINT32;
  else if (dtype == kTensorMapU64) dt = CU_TENSOR_MAP_DATA_TYPE_UINT64;
  else return SPARTA_ERR_UNSUPPORTED;
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i + 1 < rank) {
      s[i] = strides_bytes[i];
      if (s[i] % 16) return SPARTA_ERR_ALIGN;
    }
  }
  auto encode = [&] {
    return fn(map, dt, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // A thread that has made no runtime call yet that needs the device (an autograd worker thread running a
    // backward kernel) has no driver context bound; the runtime binds the primary one on such a call.
    cudaFree(nullptr);
    r = encode();
  }
  if (r != CUDA_SUCCESS && std::getenv("SPARTA_B200_DEBUG"))
    std::fprintf(stderr, "sparta_b200: cuTensorMapEncodeTiled -> %d (base %p, rank %d, dims %llu x %llu, pitch %llu, box %u x %u)\n",
                 (int)r, base, rank, (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)s[0], b[0], b[1]);
  return r == CUDA_SUCCESS ? SPARTA_OK : SPARTA_ERR_DRIVER;
}

int32_t* device_status_ptr() {
  void* p = nullptr;
  if (cudaError_t e = cudaGetSymbolAddress(&p, g_status); e != cudaSuccess) {
    if (std::getenv("SPARTA_B200_DEBUG")) std::fprintf(stderr, "sparta_b200: cudaGetSymbolAddress -> %d\n", (int)e);
    return nullptr;
  }
  return static_cast<int32_t*>(p);
}

int read_and_clear_status(int32_t out[4]) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_status, sizeof(int32_t) * 4);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int32_t zero[4] = {0, 0, 0, 0};
  e = cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  return e == cudaSuccess ? SPARTA_OK : static_cast<int>(e);
}

}  // namespace tc
}  // namespace sparta

// Reads (and clears) the status words of the current device: all zero unless a kernel's bounded wait
// ran out.  Synchronises the device.  No counterpart in the reference, whose kernels have no waits.
extern "C" int sparta_last_status(int32_t h_out[4]) {
  if (!h_out) return SPARTA_ERR_BAD_ARG;
  return sparta::tc::read_and_clear_status(h_out);
}
