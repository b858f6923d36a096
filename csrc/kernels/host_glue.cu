// Host-side glue shared by all kernels of the library: the driver entry point
// for TMA descriptor encoding (resolved at run time so the library carries no
// link-time dependency on libcuda and can be imported on a machine without a
// GPU), the device status word that bounded waits report into, and the SM count.
#include "api.h"
#include <cuda_runtime.h>
#include <stdlib.h>

namespace nkb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 tensor map with 128-byte swizzle; dims/box are innermost-first,
// strides_bytes has rank-1 entries (dimension 0 is contiguous).
int encode_tmap_bf16(CUtensorMap* m, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn || rank < 1 || rank > 5) return -1;
  cuuint64_t d[5], s[5];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i + 1 < rank) s[i] = strides_bytes[i];
  }
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, cuuint32_t(rank), const_cast<void*>(ptr), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(r);
}

int encode_tmap_bf16_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                        uint32_t box_inner, uint32_t box_outer) {
  const uint64_t dims[2] = {inner, outer};
  const uint64_t strides[1] = {ld_elems * 2};
  const uint32_t box[2] = {box_inner, box_outer};
  return encode_tmap_bf16(m, ptr, 2, dims, strides, box);
}

static int* g_status = nullptr;
static int g_num_sms = 0;
static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
int* status_word() { return g_status; }
int num_sms() { return g_num_sms; }

}  // namespace nkb

using namespace nkb;

extern "C" int nkb_init() {
  if (const char* e = getenv("NKIPY_B200_PDL")) g_pdl = atoi(e) != 0;
  if (!g_status) {
    if (cudaMalloc(&g_status, 64) != cudaSuccess) return -1;
    cudaMemset(g_status, 0, 64);
  }
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  return get_encode_fn() ? 0 : -2;
}

extern "C" void nkb_set_pdl(int enabled) { g_pdl = enabled != 0; }

extern "C" int nkb_status(int reset) {
  if (!g_status) return 0;
  int v = 0;
  cudaMemcpy(&v, g_status, sizeof(int), cudaMemcpyDeviceToHost);
  if (reset && v) cudaMemset(g_status, 0, sizeof(int));
  return v;
}
