// temporary: entry points still to be written
#include "nsa_common.cuh"
using namespace nsa;
#define STUB(name, T) extern "C" int name(const T*, void*) { set_error(#name ": not implemented yet"); return NSA_ERR_UNSUPPORTED_SHAPE; }
STUB(nsa_cmp_attn_bwd, NsaAttnParams)
STUB(nsa_swa_bwd, NsaAttnParams)
STUB(nsa_slc_attn_bwd, NsaAttnParams)
STUB(nsa_k2q_index, NsaK2qParams)
