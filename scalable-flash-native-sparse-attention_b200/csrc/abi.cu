// Error reporting and version of the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include "tma.cuh"

namespace nsa {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// cudaPeekAtLastError keeps a sticky fault visible to the caller's own checks as well.
int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
    return NSA_ERR_CUDA;
  }
  return NSA_OK;
}

int check_attn_common(const NsaAttnParams* p, const char* name, bool need_y) {
  NSA_REQUIRE(p && p->q && p->k && p->v && p->o, NSA_ERR_BAD_ARG, "%s: null tensor pointer", name);
  NSA_REQUIRE(p->meta.piece_cu && p->meta.x_cu && (!need_y || p->meta.y_cu), NSA_ERR_BAD_ARG, "%s: null metadata pointer", name);
  NSA_REQUIRE(p->D == 64 || p->D == 128, NSA_ERR_UNSUPPORTED_SHAPE, "%s: head dim %d not supported (64 or 128, qk dim == v dim)", name, p->D);
  NSA_REQUIRE(p->KH > 0 && p->QH % p->KH == 0, NSA_ERR_BAD_ARG, "%s: QH=%d must be a multiple of KH=%d", name, p->QH, p->KH);
  NSA_REQUIRE(p->QH / p->KH <= 128, NSA_ERR_UNSUPPORTED_SHAPE, "%s: more than 128 query heads per kv head", name);
  NSA_REQUIRE(p->hp.kernel_size > 0 && p->hp.stride > 0, NSA_ERR_BAD_ARG, "%s: bad kernel_size/stride", name);
  NSA_REQUIRE(!(p->meta.kv_table || p->meta.cmp_table) || (p->meta.page_size > 0 && (p->meta.page_size & (p->meta.page_size - 1)) == 0),
              NSA_ERR_UNSUPPORTED_SHAPE, "%s: page_size=%d must be a power of two", name, p->meta.page_size);
  return NSA_OK;
}

namespace tma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

bool make_map(CUtensorMap* m, const void* base, int64_t rows, int heads, int D, int64_t row_stride_elems, int box_rows, int box_heads) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || rows <= 0 || box_rows > 256 || box_heads > 256) return false;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)row_stride_elems * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
#ifdef NSA_F16
  const CUtensorMapDataType elem = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;   // matters for the bulk tensor REDUCTIONS (adds in this type)
#else
  const CUtensorMapDataType elem = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
#endif
  return fn(m, elem, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tma

}  // namespace nsa

extern "C" const char* nsa_last_error(void) { return nsa::g_err; }
extern "C" int nsa_version(void) { return 100; }
extern "C" int nsa_element_type(void) {
#ifdef NSA_F16
  return 1;
#else
  return 0;
#endif
}

extern "C" int nsa_struct_size(const char* name) {
  if (!name) return 0;
#define NSA_SZ(T) if (!strcmp(name, #T)) return (int)sizeof(T)
  NSA_SZ(NsaSeqMeta);
  NSA_SZ(NsaHyper);
  NSA_SZ(NsaPoolParams);
  NSA_SZ(NsaBlockParams);
  NSA_SZ(NsaActParams);
  NSA_SZ(NsaAttnParams);
  NSA_SZ(NsaTopkParams);
  NSA_SZ(NsaK2qParams);
  NSA_SZ(NsaCombineParams);
  NSA_SZ(NsaReorderParams);
  NSA_SZ(NsaRopeParams);
  NSA_SZ(NsaStoreKvParams);
  NSA_SZ(NsaPagedPoolParams);
  NSA_SZ(NsaDecodeParams);
  NSA_SZ(NsaWgradParams);
#undef NSA_SZ
  return 0;
}
