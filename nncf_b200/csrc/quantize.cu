// nncfb_quantize: argument validation and dispatch (see include/nncf_b200.h).
#include "quantize_launch.cuh"

using namespace nncfb;

extern "C" int nncfb_quantize(const nncfb_quantize_args* p, void* stream) {
  NNCFB_CHECK_ARG(p != nullptr, NNCFB_E_BAD_ARG, "nncfb_quantize: args is null");
  NNCFB_CHECK_ARG(p->weight != nullptr, NNCFB_E_BAD_ARG, "nncfb_quantize: weight is null");
  NNCFB_CHECK_ARG(p->outer > 0 && p->reduce > 0 && p->inner > 0, NNCFB_E_BAD_ARG,
                  "nncfb_quantize: non-positive shape [%lld, %lld, %lld]", (long long)p->outer, (long long)p->reduce,
                  (long long)p->inner);
  NNCFB_CHECK_ARG(p->mode >= NNCFB_INT8_SYM && p->mode <= NNCFB_MXFP8_E4M3, NNCFB_E_BAD_ARG,
                  "nncfb_quantize: unknown mode %d", p->mode);
  NNCFB_CHECK_ARG(p->weight_dtype == NNCFB_F32 || p->weight_dtype == NNCFB_F16 || p->weight_dtype == NNCFB_BF16,
                  NNCFB_E_BAD_ARG, "nncfb_quantize: unsupported weight dtype %d", p->weight_dtype);
  NNCFB_CHECK_ARG(p->group_size > 0, NNCFB_E_BAD_ARG, "nncfb_quantize: group_size must be positive, got %lld",
                  (long long)p->group_size);
  NNCFB_CHECK_ARG(p->reduce % p->group_size == 0, NNCFB_E_GROUP_SIZE,
                  "Channel size %lld should be divisible by size of group %lld.", (long long)p->reduce,
                  (long long)p->group_size);
  NNCFB_CHECK_ARG(p->codes_format >= NNCFB_CODES_NONE && p->codes_format <= NNCFB_CODES_NIBBLE, NNCFB_E_BAD_ARG,
                  "nncfb_quantize: bad codes_format %d", p->codes_format);
  NNCFB_CHECK_ARG(p->codes_format == NNCFB_CODES_NONE || p->codes_out != nullptr, NNCFB_E_BAD_ARG,
                  "nncfb_quantize: codes_out is null");
  const bool asym = mode_is_asym(p->mode);
  if (asym) {
    // reference: both or neither for asymmetric modes (WC/weight_lowering.py:472-477)
    NNCFB_CHECK_ARG((p->pre_scale == nullptr) == (p->pre_zp == nullptr), NNCFB_E_BAD_ARG,
                    "If precomputed quantization parameters are provided, both scale and zero point are required "
                    "for asymmetric quantization.");
    NNCFB_CHECK_ARG(p->pre_zp == nullptr || p->pre_zp_dtype == NNCFB_I32 || p->pre_zp_dtype == NNCFB_F32,
                    NNCFB_E_BAD_ARG, "nncfb_quantize: pre_zp_dtype must be NNCFB_I32 or NNCFB_F32");
  }
  const int64_t total = p->outer * p->reduce * p->inner;
  if (p->codes_format == NNCFB_CODES_NIBBLE) {
    NNCFB_CHECK_ARG(mode_bits(p->mode) == 4, NNCFB_E_BAD_ARG, "nncfb_quantize: nibble output needs a 4-bit mode");
    NNCFB_CHECK_ARG(total % 2 == 0, NNCFB_E_UNSUPPORTED, "nncfb_quantize: nibble output needs an even element count");
    if (p->inner > 1) {
      NNCFB_CHECK_ARG(p->inner % 2 == 0, NNCFB_E_UNSUPPORTED,
                      "nncfb_quantize: nibble output with inner > 1 needs an even inner size; use byte codes and "
                      "nncfb_pack_nibbles");
    } else {
      NNCFB_CHECK_ARG(p->group_size % 2 == 0, NNCFB_E_UNSUPPORTED,
                      "nncfb_quantize: nibble output needs an even group size; use byte codes and nncfb_pack_nibbles");
    }
  }

  QArgs a;
  a.weight = p->weight;
  a.pre_scale = p->pre_scale;
  a.pre_zp = asym ? p->pre_zp : nullptr;
  a.pre_zp_f32 = p->pre_zp_dtype == NNCFB_F32;
  a.codes = static_cast<uint8_t*>(p->codes_out);
  a.codes_format = p->codes_format;
  a.scale_out = p->scale_out;
  a.zp_out = p->zp_out;
  a.scale_f16 = p->scale_f16_out;
  a.scale_e8m0 = p->scale_e8m0_out;
  a.values = p->values_out;
  a.dq = p->dq_out;
  a.sqerr = p->sqerr_out;
  a.group_size = p->group_size;
  a.groups_per_row = p->reduce / p->group_size;
  a.inner = p->inner;
  a.n_groups = p->outer * a.groups_per_row * p->inner;
  a.lanes_per_group = static_cast<int>(p->group_size / 8);

  const bool aligned = aligned16(p->weight) && aligned16(p->codes_out) && aligned16(p->values_out) &&
                       aligned16(p->dq_out);
  const QuantPath path = choose_path(p->group_size, p->inner, aligned);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (p->weight_dtype) {
    case NNCFB_F32: return launch_quantize_f32(a, p->mode, path, st);
    case NNCFB_F16: return launch_quantize_f16(a, p->mode, path, st);
    default: return launch_quantize_bf16(a, p->mode, path, st);
  }
}
