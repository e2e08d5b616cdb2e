// paged_attention: operator glue for the B200 plugin (decode path).
//
// Mirrors the eager entry of the reference,
// ops/c_api/paged_attention/paged_attention_pynative.cc:649-741:
//   input_format check -> parameter / shape / type checks (:263-278, :430-506, :510-566,
//   same rules as the graph-mode twins in paged_attention_graph.cc:36-620) ->
//   context_lens read on the host (:683-692) -> param update on changed lengths
//   (:575-598) -> output like query (:712-720) -> kernel create / tiling / launch.
// Here "tiling" is the split-KV plan of libmsco_b200.so, cached by a hash of the
// attributes, shapes and context_lens, and the launch is msco_paged_attention_launch.
//
// Every combination the reference accepts is validated with the same rules;
// the combinations that are not built for B200 (listed in CheckBuiltForB200)
// fail with an "unsupported" error that names the argument.
#include <algorithm>
#include <cmath>

#include "ms_custom_ops_c.h"
#include "ops/c_api/paged_attention/paged_attention_common.h"
#include "ops/framework/module.h"
#include "ops/framework/plan_cache.h"
#include "ops/framework/tensor.h"

namespace ms_custom_ops {
namespace {

constexpr const char *kOpName = "PagedAttention";

struct PaInputs {
  Tensor query, key_cache, value_cache, block_tables, context_lens, attn_mask, batch_run_status, k_descale,
      k_offset, v_descale, v_offset, razor_offset, p_scale, log_n, q_seq_lens;
  const MsPagedAttentionArgs *a;
};

PaInputs Unpack(const MsPagedAttentionArgs *a) {
  if (a == nullptr) MS_VALUE_ERROR << "For " << kOpName << ", the argument block is NULL.";
  PaInputs in;
  in.a = a;
  in.query = Tensor(a->query);
  in.key_cache = Tensor(a->key_cache);
  in.value_cache = Tensor(a->value_cache);
  in.block_tables = Tensor(a->block_tables);
  in.context_lens = Tensor(a->context_lens);
  in.attn_mask = GetTensorOrEmpty(a->attn_mask);
  in.batch_run_status = GetTensorOrEmpty(a->batch_run_status);
  in.k_descale = GetTensorOrEmpty(a->k_descale);
  in.k_offset = GetTensorOrEmpty(a->k_offset);
  in.v_descale = GetTensorOrEmpty(a->v_descale);
  in.v_offset = GetTensorOrEmpty(a->v_offset);
  in.razor_offset = GetTensorOrEmpty(a->razor_offset);
  in.p_scale = GetTensorOrEmpty(a->p_scale);
  in.log_n = GetTensorOrEmpty(a->log_n);
  in.q_seq_lens = GetTensorOrEmpty(a->q_seq_lens);
  if (!in.query.defined() || !in.key_cache.defined() || !in.value_cache.defined() || !in.block_tables.defined() ||
      !in.context_lens.defined())
    MS_VALUE_ERROR << "For " << kOpName
                   << ", query, key_cache, value_cache, block_tables and context_lens are required.";
  return in;
}

// ---- parameter rules (reference: paged_attention_pynative.cc:34-278) -------------------------
void CheckParams(const MsPagedAttentionArgs &a) {
  const bool brs = a.batch_run_status_enable != 0;
  // head numbers
  if (a.q_head_num <= 0)
    MS_VALUE_ERROR << "For PagedAttention the q_head_num should be greater than 0, but got " << a.q_head_num << ".";
  if (a.kv_head_num < 0)
    MS_VALUE_ERROR << "For PagedAttention the kv_head_num should be greater than or equal to 0, but got "
                   << a.kv_head_num << ".";
  if (a.kv_head_num != 0 && a.q_head_num % a.kv_head_num != 0)
    MS_VALUE_ERROR << "For PagedAttention the q_head_num must be divisible by kv_head_num, but got q_head_num="
                   << a.q_head_num << ", kv_head_num=" << a.kv_head_num << ".";
  // scale type / logn
  if (!(a.scale_type >= kScaleTor && a.scale_type < kScaleMax))
    MS_VALUE_ERROR << "For PagedAttention the scale_type is invalid, got " << a.scale_type << ".";
  if (a.scale_type == kScaleLogN) {
    if (a.quant_type != kQuantUnquant)
      MS_VALUE_ERROR << "In PA scale type logn mode, quant_type must be 0(TYPE_QUANT_UNQUANT), but got "
                     << a.quant_type << ".";
    if (a.calc_type != kCalcDefault)
      MS_VALUE_ERROR << "In PA scale type logn mode, calc_type feature is not supported, but got calc_type="
                     << a.calc_type << ".";
    if (a.compress_type != kCompressNone)
      MS_VALUE_ERROR << "In PA scale type logn mode, compress_type feature is not supported, but got compress_type="
                     << a.compress_type << ".";
  }
  // MLA value head size
  if (!(a.mla_v_dim >= 0 && a.mla_v_dim <= 576))
    MS_VALUE_ERROR << "For PagedAttention(MLA mode) the value head size should be in [0, 576], but got "
                   << a.mla_v_dim << ".";
  // layout and calc type
  if (!(a.input_layout == kLayoutBSND || a.input_layout == kLayoutBNSD))
    MS_VALUE_ERROR << "For PagedAttention the input layout should be 0(BSND)/1(BNSD), but got " << a.input_layout
                   << ".";
  if (!(a.calc_type == kCalcDefault || a.calc_type == kCalcSpec))
    MS_VALUE_ERROR << "For PagedAttention the calc_type should be 0(disable MTP)/1(enable MTP), but got "
                   << a.calc_type << ".";
  if (a.calc_type == kCalcSpec) {
    if (a.quant_type != kQuantUnquant)
      MS_VALUE_ERROR << "In PA MTP scene, quant mode should be 0(TYPE_QUANT_UNQUANT), but now got " << a.quant_type
                     << ".";
    if (brs) MS_VALUE_ERROR << "In PA MTP scene, batch_run_status_enable should be false, but now got true.";
    if (a.compress_type != kCompressNone)
      MS_VALUE_ERROR << "In PA MTP scene, compress_type should be 0, but now got " << a.compress_type << ".";
  }
  if (a.input_layout == kLayoutBNSD) {
    if (a.calc_type != kCalcDefault)
      MS_VALUE_ERROR << "For PagedAttention when input layout is BNSD, calc_type feature is not supported, but got "
                     << a.calc_type << ".";
    if (a.compress_type != kCompressNone)
      MS_VALUE_ERROR << "For PagedAttention when input layout is BNSD, compress_type feature is not supported, "
                     << "but got " << a.compress_type << ".";
    if (a.quant_type != kQuantUnquant)
      MS_VALUE_ERROR << "For PagedAttention when input layout is BNSD, quant_type must be 0, but got "
                     << a.quant_type << ".";
    if (a.scale_type != kScaleTor)
      MS_VALUE_ERROR << "For PagedAttention when input layout is BNSD, scale_type must be 0, but got "
                     << a.scale_type << ".";
  }
  // compression
  if (a.compress_type == kCompressMax)
    MS_VALUE_ERROR << "In PA compress scene, compress type should not be 3(kPA_COMPRESS_TYPE_MAX).";
  if ((a.compress_type == kCompressKvHead || a.compress_type == kCompressKvHeadRope) &&
      a.quant_type != kQuantUnquant)
    MS_VALUE_ERROR << "In PA compress scene, quant_type must be 0(TYPE_QUANT_UNQUANT), but now got " << a.quant_type
                   << ".";
  if (a.compress_type == kCompressKvHeadRope) {
    if (brs)
      MS_VALUE_ERROR << "In PA COMPRESS_TYPE_KVHEAD_ROPE scene, batch_run_status_enable must be false, "
                     << "but now got true.";
    if (a.mask_type == kMaskUndefined)
      MS_VALUE_ERROR << "In PA COMPRESS_TYPE_KVHEAD_ROPE scene, mask type should not be 0(PA_MASK_UNDEFINED).";
  }
  // quantisation
  if (a.quant_type == kQuantDequantFusion && a.calc_type != kCalcDefault)
    MS_VALUE_ERROR << "For PagedAttention when quant_type is DEQUANT_FUSION, calc_type feature is not supported, "
                   << "but got " << a.calc_type << ".";
  if (a.quant_type == kQuantQkvOffline || a.quant_type == kQuantQkvOnline) {
    if (!(a.out_data_type == kOutFloat16 || a.out_data_type == kOutBFloat16))
      MS_VALUE_ERROR << "In PA full quant scene, out_data_type must be 1(Float16) or 27(BFloat16), but got "
                     << a.out_data_type << ".";
    if (a.has_quant_offset) MS_VALUE_ERROR << "In PA full quant scene, has_quant_offset must be false, but now got true.";
    if (a.compress_type != kCompressNone)
      MS_VALUE_ERROR << "In PA full quant scene, compress_type should be 0, but now got " << a.compress_type << ".";
    if (a.calc_type != kCalcDefault)
      MS_VALUE_ERROR << "In PA full quant scene, calc_type feature is not supported, but got " << a.calc_type << ".";
  }
  // MLA mode
  if (a.mla_v_dim > 0) {
    if (a.mask_type == kMaskAlibi)
      MS_VALUE_ERROR << "In PA MLA mode, mask type kPA_MASK_TYPE_ALIBI is not supported, but now got " << a.mask_type
                     << ".";
    if (a.compress_type != kCompressNone)
      MS_VALUE_ERROR << "In PA MLA mode, compress_type should be 0, but now got " << a.compress_type << ".";
    if (a.quant_type == kQuantDequantFusion)
      MS_VALUE_ERROR << "In PA MLA mode, quant_type kPA_TYPE_DEQUANT_FUSION is not supported, but now got "
                     << a.quant_type << ".";
    if (a.scale_type != kScaleTor)
      MS_VALUE_ERROR << "In PA MLA mode, scale_type must be 0(kPA_SCALE_TYPE_TOR), but now got " << a.scale_type << ".";
    if (a.input_layout != kLayoutBSND)
      MS_VALUE_ERROR << "In PA MLA mode, input layout must be 0(BSND), but now got " << a.input_layout << ".";
    if (a.kv_head_num != 1)
      MS_VALUE_ERROR << "In PA MLA mode, kv_head_num should be 1 (MQA), but now got " << a.kv_head_num << ".";
    if (a.calc_type == kCalcSpec) {
      if (a.mask_type == kMaskNorm)
        MS_VALUE_ERROR << "In PA MLA MTP scene, mask type kPA_MASK_TYPE_NORM is not supported, but now got "
                       << a.mask_type << ".";
      if (a.quant_type != kQuantUnquant)
        MS_VALUE_ERROR << "In PA MLA MTP scene, quant_type must be 0, but now got " << a.quant_type << ".";
      if (brs) MS_VALUE_ERROR << "In PA MLA MTP scene, batch_run_status_enable should be false, but now got true.";
    }
  }
}

// ---- shape rules (reference: paged_attention_pynative.cc:280-506) -------------------------------
void CheckShapes(const PaInputs &in) {
  const MsPagedAttentionArgs &a = *in.a;
  const bool nz = a.input_format == kFormatNZ;
  const size_t q_rank = nz ? 2 : kPaQueryRank, c_rank = nz ? 3 : kPaCacheRank;
  if (in.query.rank() != q_rank)
    MS_VALUE_ERROR << "For PagedAttention the rank of query must be " << q_rank << ", but got " << in.query.rank()
                   << ".";
  if (in.key_cache.rank() != c_rank)
    MS_VALUE_ERROR << "For PagedAttention the rank of key_cache must be " << c_rank
                   << " (3 for 310P/NZ, 4 for 910B/ND), but got " << in.key_cache.rank() << ".";
  if (in.value_cache.rank() != c_rank)
    MS_VALUE_ERROR << "For PagedAttention the rank of value_cache must be " << c_rank
                   << " (3 for 310P/NZ, 4 for 910B/ND), but got " << in.value_cache.rank() << ".";
  if (in.block_tables.rank() != kPaBlockTableRank)
    MS_VALUE_ERROR << "For PagedAttention the rank of block table must be " << kPaBlockTableRank << ", but got "
                   << in.block_tables.rank() << ".";
  if (in.context_lens.rank() != kPaContextLenRank)
    MS_VALUE_ERROR << "For PagedAttention the rank of context len must be " << kPaContextLenRank << ", but got "
                   << in.context_lens.rank() << ".";
  if (nz) return;
  // input_layout 0 (BSND): caches are (num_blocks, block_size, kv_heads, head_size); input_layout 1 (BNSD):
  // (num_blocks, kv_heads, block_size, head_size), the cache layout reshape_and_cache_npd writes
  // (ops/ascendc/ms_glue/reshape_and_cache_npd/reshape_and_cache_npd.md:24-25)
  const bool bnsd = a.input_layout == kLayoutBNSD;
  const int bs_dim = bnsd ? 2 : 1, h_dim = bnsd ? 1 : 2;
  const int64_t nbk = in.key_cache.dim(0), bsk = in.key_cache.dim(bs_dim), hk = in.key_cache.dim(h_dim),
                dk = in.key_cache.dim(3);
  const int64_t nbv = in.value_cache.dim(0), bsv = in.value_cache.dim(bs_dim), hv = in.value_cache.dim(h_dim),
                dv = in.value_cache.dim(3);
  if (a.mla_v_dim == 0) {
    if (nbk != nbv)
      MS_VALUE_ERROR << "For PagedAttention the num_blocks of key_cache and value_cache must be same, but got " << nbk
                     << " and " << nbv << ".";
    if (bsk != bsv)
      MS_VALUE_ERROR << "For PagedAttention the block_size of key_cache and value_cache must be same, but got " << bsk
                     << " and " << bsv << ".";
    if (hk != hv)
      MS_VALUE_ERROR << "For PagedAttention the head_num of key_cache and value_cache must be same, but got " << hk
                     << " and " << hv << ".";
  }
  if (dk != in.query.dim(2))
    MS_VALUE_ERROR << "For PagedAttention the head_size of key_cache and query must be same, but got " << dk << " and "
                   << in.query.dim(2) << ".";
  if (a.mla_v_dim == 0) {
    if (!(dk > 0 && dk <= 256))
      MS_VALUE_ERROR << "For PagedAttention on ND path, head_size of key_cache must be in (0, 256], but got " << dk
                     << ".";
    if (bsk * dk > 128 * 128)
      MS_VALUE_ERROR << "For PagedAttention on ND path, block_size * head_size must be <= 128 * 128, but got "
                     << bsk * dk << ".";
  } else {
    if (!(dk <= 576 && dv <= 576))
      MS_VALUE_ERROR << "For PagedAttention MLA mode, head_size of key_cache and value_cache must be <= 576, but got "
                     << dk << " and " << dv << ".";
    if ((dk > 256 || dv > 256) && bsk > 128)
      MS_VALUE_ERROR << "For PagedAttention MLA mode, when head_size > 256, block_size must be <= 128, but got "
                     << "head_size_k=" << dk << ", head_size_v=" << dv << ", block_size=" << bsk << ".";
  }
  if (a.mask_type == kMaskFree)
    MS_VALUE_ERROR << "For PagedAttention, MASK_FREE is only supported on 310P (NZ format).";
}

// ---- dtype rules (reference: paged_attention_pynative.cc:510-566) --------------------------------
void CheckTypes(const PaInputs &in) {
  const int32_t q = in.query.dtype(), k = in.key_cache.dtype(), v = in.value_cache.dtype();
  const int64_t qt = in.a->quant_type;
  auto is_half = [](int32_t t) { return t == MSCO_DTYPE_F16 || t == MSCO_DTYPE_BF16; };
  if (qt == kQuantUnquant) {
    if (!is_half(q))
      MS_VALUE_ERROR << "For PagedAttention in unquant mode, query dtype must be float16/bfloat16, but got type: "
                     << DTypeName(q) << ".";
    if (!is_half(k))
      MS_VALUE_ERROR << "For PagedAttention in unquant mode, key cache dtype must be float16/bfloat16, but got type: "
                     << DTypeName(k) << ".";
    if (!is_half(v))
      MS_VALUE_ERROR << "For PagedAttention in unquant mode, value cache dtype must be float16/bfloat16, "
                     << "but got type: " << DTypeName(v) << ".";
  } else if (qt == kQuantDequantFusion) {
    if (!is_half(q))
      MS_VALUE_ERROR << "For PagedAttention in dequant mode, query dtype must be float16/bfloat16, but got type: "
                     << DTypeName(q) << ".";
    if (k != MSCO_DTYPE_I8)
      MS_VALUE_ERROR << "For PagedAttention in dequant mode, key cache dtype must be int8, but got type: "
                     << DTypeName(k) << ".";
    if (v != MSCO_DTYPE_I8)
      MS_VALUE_ERROR << "For PagedAttention in dequant mode, value cache dtype must be int8, but got type: "
                     << DTypeName(v) << ".";
  } else if (qt == kQuantQkvOffline || qt == kQuantQkvOnline) {
    if (q != MSCO_DTYPE_I8)
      MS_VALUE_ERROR << "For PagedAttention in full quant mode, query dtype must be int8, but got type: "
                     << DTypeName(q) << ".";
    if (k != MSCO_DTYPE_I8 || v != MSCO_DTYPE_I8)
      MS_VALUE_ERROR << "For PagedAttention in full quant mode, key/value cache dtype must be int8.";
  }
}

// ---- what this build implements ------------------------------------------------------------------
void CheckBuiltForB200(const PaInputs &in) {
  const MsPagedAttentionArgs &a = *in.a;
  if (a.input_format == kFormatNZ)
    MS_UNSUPPORTED << "For PagedAttention, input_format=1 (FRACTAL_NZ, Ascend 310P) is not built for B200; use 0 (ND).";
  if (a.quant_type == kQuantQkvOffline || a.quant_type == kQuantQkvOnline)
    MS_UNSUPPORTED << "For PagedAttention, quant_type=" << a.quant_type
                   << " (full int8 QKV) is not built for B200; quant_type 0 and 1 are.";
  if (a.quant_type != kQuantUnquant && a.quant_type != kQuantDequantFusion)
    MS_VALUE_ERROR << "For PagedAttention, quant_type is invalid, got " << a.quant_type << ".";
  if (a.mask_type < 0 || a.mask_type > kMaskFree)
    MS_VALUE_ERROR << "For PagedAttention, mask_type is invalid, got " << a.mask_type << ".";
  if (a.mask_type == kMaskFree || (a.mask_type == kMaskSpec && a.calc_type != kCalcSpec))
    MS_UNSUPPORTED << "For PagedAttention, mask_type=" << a.mask_type << " is not built for B200; mask_type 0 (none), "
                   << "1 (NORM), 2 (ALIBI), and 3 (SPEC) together with calc_type=1 are.";
  if (a.calc_type == kCalcSpec && (a.mask_type == kMaskNorm || a.mask_type == kMaskAlibi))
    MS_UNSUPPORTED << "For PagedAttention, calc_type=1 (multi-token queries) is built for B200 with mask_type 0 "
                   << "(none) or 3 (SPEC); the prefill-shaped NORM / ALIBI masks are not.";
  if (a.compress_type != kCompressNone)
    MS_UNSUPPORTED << "For PagedAttention, compress_type=" << a.compress_type << " is not built for B200.";
  if (a.scale_type != kScaleTor)
    MS_UNSUPPORTED << "For PagedAttention, scale_type=1 (LogN) is not built for B200.";
  if (a.mla_v_dim != 0)
    MS_UNSUPPORTED << "For PagedAttention, mla_v_dim>0 (MLA mode) is not built for B200.";
  if (a.batch_run_status_enable)
    MS_UNSUPPORTED << "For PagedAttention, batch_run_status_enable=True is not built for B200.";
}

struct Prepared {
  MscoPaDesc desc;
  std::vector<int32_t> context_lens;  // one per row of the decode batch (per query token with calc_type = 1)
  int64_t batch = 0;                  // rows of the decode batch = query.dim(0)
  // calc_type = 1 (multi-token queries): every query token is a row of the decode batch that shares
  // the block table and the context length of its sequence (paged_attention_graph.cc:758-762, q_seq_len)
  bool multi_token = false;
  std::vector<int32_t> seq_of_row;  // sequence (row of block_tables) of every query token
  // ... unless the kernel library can stack the tokens of a sequence into the q rows of its work items
  // (one read of the context for all of them): then the plan is made from the per-sequence lengths
  bool stacked = false;
  std::vector<int32_t> seq_lens, q_lens;  // one entry per sequence (multi_token only)
};

// Bytes behind the plan's workspace that hold the per-token block table and its row index.
size_t TokenTableBytes(const Prepared &p) {
  if (!p.multi_token || p.stacked) return 0;
  const size_t cells = static_cast<size_t>(p.batch) * static_cast<size_t>(p.desc.max_blocks_per_seq);
  return (cells * 4 + 255) / 256 * 256 + (static_cast<size_t>(p.batch) * 4 + 255) / 256 * 256;
}

Prepared Prepare(const PaInputs &in) {
  const MsPagedAttentionArgs &a = *in.a;
  if (a.input_format != kFormatND && a.input_format != kFormatNZ)
    MS_RUNTIME_ERROR << "For " << kOpName << ", the input_format is invalid: " << a.input_format;
  CheckParams(a);
  CheckShapes(in);
  CheckTypes(in);
  CheckBuiltForB200(in);

  Prepared p;
  p.context_lens = GetInt32VectorFromHostTensor(in.context_lens, kOpName, "context_lens");
  p.batch = in.query.dim(0);
  const int64_t num_seqs = static_cast<int64_t>(p.context_lens.size());
  if (a.calc_type == kCalcSpec) {
    if (!in.q_seq_lens.defined())
      MS_RUNTIME_ERROR << "For " << kOpName << ", calc_type is SPEC(MTP), q_seq_lens must be provided.";
    const std::vector<int32_t> q_lens = GetInt32VectorFromHostTensor(in.q_seq_lens, kOpName, "q_seq_lens");
    if (static_cast<int64_t>(q_lens.size()) != num_seqs)
      MS_VALUE_ERROR << "For PagedAttention, q_seq_lens has " << q_lens.size() << " entries but context_lens has "
                     << num_seqs << ".";
    std::vector<int32_t> per_token;
    for (int64_t b = 0; b < num_seqs; ++b) {
      if (q_lens[b] < 0) MS_VALUE_ERROR << "For PagedAttention, q_seq_lens must not be negative, but got " << q_lens[b] << ".";
      for (int32_t t = 0; t < q_lens[b]; ++t) {
        p.seq_of_row.push_back(static_cast<int32_t>(b));
        per_token.push_back(p.context_lens[b]);
      }
    }
    if (static_cast<int64_t>(per_token.size()) != p.batch)
      MS_VALUE_ERROR << "For PagedAttention, q_seq_lens sum to " << per_token.size() << " but query holds " << p.batch
                     << " tokens.";
    if (in.block_tables.dim(0) != num_seqs)
      MS_VALUE_ERROR << "For PagedAttention, block_tables has " << in.block_tables.dim(0) << " rows but there are "
                     << num_seqs << " sequences.";
    p.seq_lens = p.context_lens;
    p.q_lens = q_lens;
    p.context_lens.swap(per_token);
    p.multi_token = true;
  }
  const int64_t hq = in.query.dim(1), d = in.query.dim(2);
  const bool bnsd = a.input_layout == kLayoutBNSD;
  const int64_t hkv = in.key_cache.dim(bnsd ? 1 : 2);
  if (hq != a.q_head_num)
    MS_VALUE_ERROR << "For PagedAttention the q_head_num (" << a.q_head_num << ") must equal query's head dimension ("
                   << hq << ").";
  if (a.kv_head_num != 0 && a.kv_head_num != hkv)
    MS_VALUE_ERROR << "For PagedAttention the kv_head_num (" << a.kv_head_num
                   << ") must equal the head_num of key_cache (" << hkv << ").";
  if (hq % hkv != 0)
    MS_VALUE_ERROR << "For PagedAttention the q_head_num must be divisible by the head_num of key_cache, but got "
                   << hq << " and " << hkv << ".";
  if (static_cast<int64_t>(p.context_lens.size()) != p.batch)
    MS_VALUE_ERROR << "For PagedAttention, context_lens has " << p.context_lens.size()
                   << " entries but query holds " << p.batch << " tokens (decode: one token per sequence).";
  if (!p.multi_token && in.block_tables.dim(0) != p.batch)
    MS_VALUE_ERROR << "For PagedAttention, block_tables has " << in.block_tables.dim(0) << " rows but the batch is "
                   << p.batch << ".";
  if (in.block_tables.dtype() != MSCO_DTYPE_I32)
    MS_VALUE_ERROR << "For PagedAttention, block_tables must be Int32, but got " << DTypeName(in.block_tables.dtype())
                   << ".";
  if (in.value_cache.dim(3) != d)
    MS_VALUE_ERROR << "For PagedAttention the head_size of value_cache and query must be same, but got "
                   << in.value_cache.dim(3) << " and " << d << ".";
  if (in.key_cache.dtype() != in.value_cache.dtype())
    MS_VALUE_ERROR << "For PagedAttention, key_cache and value_cache must have the same dtype.";
  if (a.quant_type == kQuantUnquant && in.key_cache.dtype() != in.query.dtype())
    MS_VALUE_ERROR << "For PagedAttention in unquant mode, the cache dtype must equal the query dtype, but got "
                   << DTypeName(in.key_cache.dtype()) << " and " << DTypeName(in.query.dtype()) << ".";
  for (const auto &nt : {std::make_pair(&in.query, "query"), std::make_pair(&in.key_cache, "key_cache"),
                         std::make_pair(&in.value_cache, "value_cache"), std::make_pair(&in.block_tables, "block_tables"),
                         std::make_pair(&in.attn_mask, "attn_mask"), std::make_pair(&in.k_descale, "k_descale"),
                         std::make_pair(&in.k_offset, "k_offset"), std::make_pair(&in.v_descale, "v_descale"),
                         std::make_pair(&in.v_offset, "v_offset")})
    CheckContiguous(*nt.first, kOpName, nt.second);

  MscoPaDesc &ds = p.desc;
  ds = MscoPaDesc();
  ds.q_dtype = in.query.dtype();
  ds.kv_dtype = in.key_cache.dtype();
  ds.num_q_heads = static_cast<int32_t>(hq);
  ds.num_kv_heads = static_cast<int32_t>(hkv);
  ds.head_dim = static_cast<int32_t>(d);
  ds.block_size = static_cast<int32_t>(in.key_cache.dim(bnsd ? 2 : 1));
  ds.cache_layout = bnsd ? 1 : 0;
  ds.num_blocks = in.key_cache.dim(0);
  ds.max_blocks_per_seq = static_cast<int32_t>(in.block_tables.dim(1));
  ds.qk_scale = static_cast<float>(a.qk_scale);
  ds.quant_type = static_cast<int32_t>(a.quant_type);
  ds.has_quant_offset = a.has_quant_offset ? 1 : 0;
  ds.mask_type = static_cast<int32_t>(a.mask_type);
  if (a.quant_type == kQuantDequantFusion) {
    auto vec = [&](const Tensor &t, const char *name, int32_t dt, bool required) {
      if (!t.defined()) {
        if (required) MS_VALUE_ERROR << "For PagedAttention in dequant mode, " << name << " must be provided.";
        return;
      }
      if (t.dtype() != dt)
        MS_VALUE_ERROR << "For PagedAttention in dequant mode, " << name << " must be " << DTypeName(dt)
                       << ", but got " << DTypeName(t.dtype()) << ".";
      if (t.numel() != hkv * d)
        MS_VALUE_ERROR << "For PagedAttention in dequant mode, " << name << " must have kv_head_num * head_size = "
                       << hkv * d << " elements, but got " << t.numel() << ".";
    };
    vec(in.k_descale, "k_descale", MSCO_DTYPE_F32, true);
    vec(in.v_descale, "v_descale", MSCO_DTYPE_F32, true);
    vec(in.k_offset, "k_offset", MSCO_DTYPE_I32, a.has_quant_offset != 0);
    vec(in.v_offset, "v_offset", MSCO_DTYPE_I32, a.has_quant_offset != 0);
  }
  if (a.mask_type != kMaskUndefined) {
    if (!in.attn_mask.defined())
      MS_VALUE_ERROR << "For PagedAttention, attn_mask must be provided when mask_type is " << a.mask_type << ".";
    const Tensor &m = in.attn_mask;
    const int64_t max_len = p.context_lens.empty() ? 0 : *std::max_element(p.context_lens.begin(), p.context_lens.end());
    if (a.mask_type == kMaskSpec) {  // [tokens, max_context]: the NORM decode mask of the per-token batch
      if (m.rank() != 2 || m.dim(0) != p.batch)
        MS_VALUE_ERROR << "For PagedAttention, the SPEC mask must have shape (num_tokens, max_context).";
      ds.mask_type = kMaskNorm;
      ds.mask_batch_stride = m.dim(1);
      ds.mask_head_stride = 0;
    } else if (a.mask_type == kMaskNorm) {  // decode: [batch, 1, max_context]
      if (m.rank() != 3 || m.dim(0) != p.batch || m.dim(1) != 1)
        MS_VALUE_ERROR << "For PagedAttention, the NORM mask of a decode step must have shape (batch, 1, max_context).";
      ds.mask_batch_stride = m.dim(2);
      ds.mask_head_stride = 0;
    } else {  // ALIBI: [batch, q_heads, 1, max_context]
      if (m.rank() != 4 || m.dim(0) != p.batch || m.dim(1) != hq || m.dim(2) != 1)
        MS_VALUE_ERROR << "For PagedAttention, the ALIBI mask of a decode step must have shape "
                       << "(batch, q_head_num, 1, max_context).";
      ds.mask_batch_stride = m.dim(1) * m.dim(3);
      ds.mask_head_stride = m.dim(3);
    }
    if (m.dim(m.rank() - 1) < max_len)
      MS_VALUE_ERROR << "For PagedAttention, the mask covers " << m.dim(m.rank() - 1)
                     << " positions but the longest context has " << max_len << ".";
    if (m.dtype() != MSCO_DTYPE_F16 && m.dtype() != MSCO_DTYPE_BF16 && m.dtype() != MSCO_DTYPE_F32)
      MS_VALUE_ERROR << "For PagedAttention, attn_mask must be float16/bfloat16/float32.";
    ds.mask_dtype = m.dtype();
  }
  p.stacked = p.multi_token && msco_paged_attention_tma_supported(&ds) != 0;
  return p;
}

PlanRef GetPlan(const Prepared &p) {
  if (p.stacked) return PlanCache::Instance().GetOrCreate(p.desc, p.seq_lens, &p.q_lens);
  return PlanCache::Instance().GetOrCreate(p.desc, p.context_lens);
}

// Workspace bytes the last launch attempt of this thread needed (see ..._last_workspace_need).
thread_local size_t g_last_workspace_need = 0;

}  // namespace
}  // namespace ms_custom_ops

MS_CUSTOM_OPS_REGISTER_OP(
    paged_attention,
    "paged_attention(query, key_cache, value_cache, block_tables, context_lens, attn_mask=None, "
    "batch_run_status=None, k_descale=None, k_offset=None, v_descale=None, v_offset=None, razor_offset=None, "
    "p_scale=None, log_n=None, q_seq_lens=None, q_head_num=0, qk_scale=1.0, kv_head_num=0, mask_type=0, "
    "batch_run_status_enable=False, quant_type=0, out_data_type=-1, has_quant_offset=False, compress_type=0, "
    "calc_type=0, scale_type=0, input_layout=0, mla_v_dim=0, input_format=0)")

extern "C" int ms_custom_ops_paged_attention_infer(const MsPagedAttentionArgs *args, int32_t *out_dtype,
                                                   int32_t *out_ndim, int64_t *out_shape) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    const PaInputs in = Unpack(args);
    (void)Prepare(in);
    if (out_dtype) *out_dtype = in.query.dtype();
    if (out_ndim) *out_ndim = static_cast<int32_t>(in.query.rank());
    if (out_shape)
      for (size_t i = 0; i < in.query.rank(); ++i) out_shape[i] = in.query.dim(i);
    return MSCO_OK;
  });
}

extern "C" int ms_custom_ops_paged_attention_workspace_size(const MsPagedAttentionArgs *args, size_t *bytes) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    const PaInputs in = Unpack(args);
    const Prepared p = Prepare(in);
    PlanRef plan = GetPlan(p);
    if (bytes)
      *bytes = (std::max<size_t>(msco_paged_attention_workspace_bytes(plan.get()), 256) + 255) / 256 * 256 +
               TokenTableBytes(p);
    return MSCO_OK;
  });
}

namespace ms_custom_ops {
namespace {

// Shared by the operator and its variant with the log-sum-exp output (lse_out undefined: none).
int LaunchPagedAttention(const MsPagedAttentionArgs *args, const Tensor &out, const Tensor &lse_out, void *workspace,
                         size_t workspace_bytes, void *stream) {
  const PaInputs in = Unpack(args);
  const Prepared p = Prepare(in);
  if (!out.defined() || out.data() == nullptr)
    MS_VALUE_ERROR << "For PagedAttention, attention_out must be allocated by the caller.";
  if (out.dtype() != in.query.dtype() || out.shape() != in.query.shape())
    MS_VALUE_ERROR << "For PagedAttention, attention_out must have query's shape and dtype.";
  CheckContiguous(out, kOpName, "attention_out");
  if (lse_out.defined()) {
    if (lse_out.dtype() != MSCO_DTYPE_F32)
      MS_TYPE_ERROR << "For PagedAttention, lse_out must be Float32, but got " << DTypeName(lse_out.dtype()) << ".";
    if (lse_out.rank() != 2 || lse_out.dim(0) != in.query.dim(0) || lse_out.dim(1) != in.query.dim(1))
      MS_VALUE_ERROR << "For PagedAttention, lse_out must be (batch, q_head_num) = (" << in.query.dim(0) << ", "
                     << in.query.dim(1) << ").";
    if (lse_out.data() == nullptr && p.batch != 0)
      MS_VALUE_ERROR << "For PagedAttention, lse_out must be allocated by the caller.";
    CheckContiguous(lse_out, kOpName, "lse_out");
  }
  if (p.batch == 0) return MSCO_OK;
  PlanRef plan = GetPlan(p);
  const size_t plan_ws = (std::max<size_t>(msco_paged_attention_workspace_bytes(plan.get()), 256) + 255) / 256 * 256;
  g_last_workspace_need = plan_ws + TokenTableBytes(p);
  if (workspace == nullptr || workspace_bytes < g_last_workspace_need)
    MS_VALUE_ERROR << "For PagedAttention, the workspace holds " << workspace_bytes << " bytes but this launch needs "
                   << g_last_workspace_need << ".";
  const int32_t *tables = static_cast<const int32_t *>(in.block_tables.data());
  if (p.multi_token && !p.stacked) {
    // one block-table row per query token, built behind the plan's part of the workspace
    const size_t cells = static_cast<size_t>(p.batch) * static_cast<size_t>(p.desc.max_blocks_per_seq);
    int32_t *token_tables = reinterpret_cast<int32_t *>(static_cast<char *>(workspace) + plan_ws);
    int32_t *row_index = reinterpret_cast<int32_t *>(static_cast<char *>(workspace) + plan_ws +
                                                     (cells * 4 + 255) / 256 * 256);
    const int rc = msco_expand_rows_i32(tables, static_cast<int32_t>(in.block_tables.dim(0)),
                                        p.desc.max_blocks_per_seq, p.seq_of_row.data(),
                                        static_cast<int32_t>(p.batch), token_tables, row_index, stream);
    if (rc != MSCO_OK) return rc;
    tables = token_tables;
  }
  workspace_bytes = plan_ws;
  const float *kd = static_cast<const float *>(in.k_descale.data());
  const float *vd = static_cast<const float *>(in.v_descale.data());
  const int32_t *ko = static_cast<const int32_t *>(in.k_offset.data());
  const int32_t *vo = static_cast<const int32_t *>(in.v_offset.data());
  if (lse_out.defined())
    return msco_paged_attention_launch_lse(plan.get(), in.query.data(), in.key_cache.data(), in.value_cache.data(),
                                           tables, kd, ko, vd, vo, in.attn_mask.data(), out.data(),
                                           static_cast<float *>(lse_out.data()), workspace, workspace_bytes, stream);
  return msco_paged_attention_launch(plan.get(), in.query.data(), in.key_cache.data(), in.value_cache.data(), tables,
                                     kd, ko, vd, vo, in.attn_mask.data(), out.data(), workspace, workspace_bytes,
                                     stream);
}

}  // namespace
}  // namespace ms_custom_ops

extern "C" int ms_custom_ops_paged_attention(const MsPagedAttentionArgs *args, const MsTensorDesc *attention_out,
                                             void *workspace, size_t workspace_bytes, void *stream) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    return LaunchPagedAttention(args, Tensor(attention_out), Tensor(), workspace, workspace_bytes, stream);
  });
}

extern "C" int ms_custom_ops_paged_attention_with_lse(const MsPagedAttentionArgs *args,
                                                      const MsTensorDesc *attention_out, const MsTensorDesc *lse_out,
                                                      void *workspace, size_t workspace_bytes, void *stream) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    const Tensor lse(lse_out);
    if (!lse.defined()) MS_VALUE_ERROR << "For PagedAttention, lse_out must be provided.";
    return LaunchPagedAttention(args, Tensor(attention_out), lse, workspace, workspace_bytes, stream);
  });
}

extern "C" size_t ms_custom_ops_paged_attention_last_workspace_need(void) {
  return ms_custom_ops::g_last_workspace_need;
}

extern "C" int ms_custom_ops_paged_attention_status(const void *workspace) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] { return msco_paged_attention_status(nullptr, workspace); });
}
