// nncfb_quantize: argument validation and dispatch (see include/nncf_b200.h).
#include "quantize_launch.cuh"

using namespace nncfb;

namespace {

int validate(const nncfb_quantize_args* p);
int launch_general(const nncfb_quantize_args* p, cudaStream_t st);

int launch_fast_run(const nncfb_quantize_args* items, int n, FastClass cls, cudaStream_t st) {
  // the descriptor table travels as a kernel parameter (no device workspace, graph-capturable)
  static thread_local FastBatch batch;
  const size_t esz = items[0].weight_dtype == NNCFB_F32 ? 4 : 2;
  batch.n_tensors = n;
  batch.codes_nibble = mode_bits(items[0].mode) == 4;
  batch.iter_start[0] = 0;
  for (int i = 0; i < n; ++i) {
    const nncfb_quantize_args& p = items[i];
    FastTensor& t = batch.t[i];
    t.weight = p.weight;
    t.codes = static_cast<uint8_t*>(p.codes_out);
    t.scale = p.scale_out;
    t.zp = p.zp_out;
    t.zp_packed = p.zp_packed_out;
    t.scale_f16 = p.scale_f16_out;
    t.e8m0 = p.scale_e8m0_out;
    t.n_groups = p.outer * (p.reduce / p.group_size);
    batch.iter_start[i + 1] = batch.iter_start[i] + fast_iterations(cls, t.n_groups, esz);
  }
  switch (items[0].weight_dtype) {
#ifndef NNCFB_ONLY_BF16  // tuning builds link the bf16 kernels only
    case NNCFB_F32: return launch_fast_f32(batch, items[0].mode, cls, st);
    case NNCFB_F16: return launch_fast_f16(batch, items[0].mode, cls, st);
#endif
    default: return launch_fast_bf16(batch, items[0].mode, cls, st);
  }
}

}  // namespace

extern "C" int nncfb_quantize_batch(const nncfb_quantize_args* items, int32_t n, void* stream) {
  NNCFB_CHECK_ARG(items != nullptr || n == 0, NNCFB_E_BAD_ARG, "nncfb_quantize_batch: items is null");
  NNCFB_CHECK_ARG(n >= 0, NNCFB_E_BAD_ARG, "nncfb_quantize_batch: negative count");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < n; ++i) {
    const int rc = validate(&items[i]);
    if (rc != NNCFB_OK) return rc;
  }
  int i = 0;
  while (i < n) {
    const FastClass cls = fast_class(items[i]);
    if (cls.kind == 0) {
      const int rc = launch_general(&items[i], st);
      if (rc != NNCFB_OK) return rc;
      ++i;
      continue;
    }
    int j = i + 1;
    while (j < n && j - i < kMaxBatchTensors && items[j].mode == items[i].mode &&
           items[j].weight_dtype == items[i].weight_dtype && fast_class(items[j]) == cls)
      ++j;
    const int rc = launch_fast_run(items + i, j - i, cls, st);
    if (rc != NNCFB_OK) return rc;
    i = j;
  }
  return NNCFB_OK;
}

extern "C" int nncfb_quantize(const nncfb_quantize_args* p, void* stream) {
  const int rc = validate(p);
  if (rc != NNCFB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const FastClass cls = fast_class(*p);
  if (cls.kind != 0) return launch_fast_run(p, 1, cls, st);
  return launch_general(p, st);
}

namespace {

int validate(const nncfb_quantize_args* p) {
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
  return NNCFB_OK;
}

int launch_general(const nncfb_quantize_args* p, cudaStream_t st) {
  const bool asym = mode_is_asym(p->mode);

  QArgs a;
  a.weight = p->weight;
  a.pre_scale = p->pre_scale;
  a.pre_zp = asym ? p->pre_zp : nullptr;
  a.pre_zp_f32 = p->pre_zp_dtype == NNCFB_F32;
  a.codes = static_cast<uint8_t*>(p->codes_out);
  a.codes_format = p->codes_format;
  a.scale_out = p->scale_out;
  a.zp_out = p->zp_out;
  a.zp_packed = asym ? p->zp_packed_out : nullptr;
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
  if (a.zp_packed != nullptr && mode_bits(p->mode) == 4) {
    // nibbles are ORed into place by whichever thread owns the group: the words start at zero
    NNCFB_CHECK_ARG((reinterpret_cast<uintptr_t>(a.zp_packed) & 3u) == 0, NNCFB_E_ALIGNMENT,
                    "nncfb_quantize: zp_packed_out must be 4-byte aligned");
    NNCFB_CUDA(cudaMemsetAsync(a.zp_packed, 0, static_cast<size_t>((a.n_groups + 7) / 8) * 4, st));
  }

  const bool aligned = aligned16(p->weight) && aligned16(p->codes_out) && aligned16(p->values_out) &&
                       aligned16(p->dq_out);
  QuantPath path = choose_path(p->group_size, p->inner, aligned);
  // Storage outputs of a column-group layout with tall groups (per-channel weights stored [in, out]) and whole
  // 16-byte column vectors: the tiled kernel.  The thread-per-column kernel has too few threads there (one per
  // column pair) and walks the group serially; for short groups it has plenty and is the faster of the two.
  if (path == QuantPath::kColumn && p->group_size >= 512 && p->inner % 8 == 0 && aligned && !p->pre_scale && !p->values_out && !p->dq_out &&
      !p->sqerr_out && (p->codes_format == NNCFB_CODES_NONE || p->codes_out)) {
    path = QuantPath::kColumnTile;
  }
  switch (p->weight_dtype) {
#ifndef NNCFB_ONLY_BF16
    case NNCFB_F32: return launch_quantize_f32(a, p->mode, path, st);
    case NNCFB_F16: return launch_quantize_f16(a, p->mode, path, st);
#endif
    default: return launch_quantize_bf16(a, p->mode, path, st);
  }
}

}  // namespace
