// Device-resident model state: weights arena, paged KV cache with its block table, GDN state pool.
// Page hand-out order, LIFO reuse and dirty-row upload follow the reference (src/kv_cache.cpp:10-88):
// page ids are part of the parity contract.
#include <algorithm>

#include "qwen38/api.h"

namespace qwen38 {

namespace {
constexpr size_t kPlaneAlign = 256;
size_t padded(int64_t bytes) { return size_t(align_up(bytes, int64_t(kPlaneAlign))); }
}  // namespace

// ---- weights ------------------------------------------------------------------------------------
size_t ModelWeights::required_device_bytes(const ModelFile& file, EmbeddingPlacement placement) {
  size_t total = kPlaneAlign;
  for (const auto& [name, t] : file.tensors()) {
    if (name == "embed" && placement == EmbeddingPlacement::Host) continue;
    total += is_bq(t.dtype) ? padded(t.lo_bytes) + padded(t.hi_bytes) + padded(t.sc_bytes) : padded(t.bytes);
  }
  return total;
}

const void* ModelWeights::upload_range(const ModelFile& file, int64_t offset, int64_t bytes) {
  if (bytes == 0) return nullptr;
  void* dst = arena_.allocate(size_t(bytes), kPlaneAlign);
  QWEN38_CUDA(cudaMemcpy(dst, file.data(offset, bytes).data(), size_t(bytes), cudaMemcpyHostToDevice));
  return dst;
}

kernels::BQWeight ModelWeights::upload_bq(const ModelFile& file, const std::string& name) {
  const TensorInfo& t = file.tensor(name);
  QWEN38_CHECK(is_bq(t.dtype), name, " must be a BQ tensor");
  kernels::BQWeight w;
  w.bits = bq_bits(t.dtype);
  w.n = int(t.shape[0]);
  w.k = int(t.shape[1]);
  w.rows = int(t.rows);
  w.lo = static_cast<const uint8_t*>(upload_range(file, t.lo_offset, t.lo_bytes));
  w.hi = static_cast<const uint8_t*>(upload_range(file, t.hi_offset, t.hi_bytes));
  w.scales = static_cast<const __nv_bfloat16*>(upload_range(file, t.sc_offset, t.sc_bytes));
  return w;
}

ModelWeights::ModelWeights(const ModelFile& file, EmbeddingPlacement placement)
    : arena_(required_device_bytes(file, placement)), placement_(placement) {
  const ModelConfig& cfg = file.config();
  const TensorInfo& emb = file.tensor("embed");
  QWEN38_CHECK(emb.dtype == DType::BF16, "embedding must be bf16");
  if (placement == EmbeddingPlacement::Host) {
    embed_host_ = PinnedBuffer(size_t(emb.bytes), true);
    std::memcpy(embed_host_.get(), file.data(emb.offset, emb.bytes).data(), size_t(emb.bytes));
    embedding_ = static_cast<const __nv_bfloat16*>(embed_host_.device_ptr());
  } else {
    embedding_ = static_cast<const __nv_bfloat16*>(upload_range(file, emb.offset, emb.bytes));
  }
  auto direct = [&](const std::string& name) {
    const TensorInfo& t = file.tensor(name);
    return upload_range(file, t.offset, t.bytes);
  };
  layers_.resize(size_t(cfg.num_layers));
  for (int i = 0; i < cfg.num_layers; ++i) {
    LayerWeights& L = layers_[size_t(i)];
    const std::string p = std::to_string(i) + ".";
    L.attention = cfg.is_attention[size_t(i)] != 0;
    if (L.attention) {
      L.in_proj = upload_bq(file, p + "attn.qkvg");
      L.out_proj = upload_bq(file, p + "attn.o");
      L.q_norm = static_cast<const float*>(direct(p + "attn.q_norm"));
      L.k_norm = static_cast<const float*>(direct(p + "attn.k_norm"));
    } else {
      L.in_proj = upload_bq(file, p + "gdn.qkvz");
      L.out_proj = upload_bq(file, p + "gdn.out");
      L.ab = static_cast<const __nv_bfloat16*>(direct(p + "gdn.ab"));
      L.ab_rows = int(file.tensor(p + "gdn.ab").shape[0]);
      L.conv = static_cast<const float*>(direct(p + "gdn.conv"));
      L.A = static_cast<const float*>(direct(p + "gdn.A"));
      L.dt_bias = static_cast<const float*>(direct(p + "gdn.dt_bias"));
      L.gdn_norm = static_cast<const float*>(direct(p + "gdn.norm"));
    }
    L.gate_up = upload_bq(file, p + "mlp.gate_up");
    L.down = upload_bq(file, p + "mlp.down");
  }
  lm_head_ = upload_bq(file, "lm_head");
}

// ---- KV cache -------------------------------------------------------------------------------------
size_t KvCache::page_bytes_all_layers(const ModelConfig& cfg, kernels::KvDtype dtype) {
  return kernels::KvCacheDesc::page_bytes_for(dtype, cfg.num_key_value_heads) * size_t(cfg.num_attention_layers());
}

KvCache::KvCache(const ModelConfig& cfg, kernels::KvDtype dtype, int num_pages, int num_slots, int max_pages_per_seq)
    : num_pages_(num_pages), num_slots_(num_slots), max_pages_per_seq_(max_pages_per_seq), dtype_(dtype),
      kv_heads_(cfg.num_key_value_heads) {
  QWEN38_CHECK(cfg.head_dim == kernels::kHeadDim, "KV cache: head_dim");
  QWEN38_CHECK(num_pages > 0 && num_slots > 0 && max_pages_per_seq > 0, "KV cache: sizes");
  page_bytes_ = kernels::KvCacheDesc::page_bytes_for(dtype, kv_heads_);
  layer_stride_ = page_bytes_ * size_t(num_pages);
  pool_ = DeviceBuffer(layer_stride_ * size_t(std::max(1, cfg.num_attention_layers())));
  QWEN38_CUDA(cudaMemset(pool_.get(), 0, pool_.bytes()));
  const size_t table_bytes = size_t(num_slots) * size_t(max_pages_per_seq) * sizeof(int);
  table_dev_ = DeviceBuffer(table_bytes);
  table_host_ = PinnedBuffer(table_bytes, false);
  std::memset(table_host_.get(), 0, table_bytes);
  QWEN38_CUDA(cudaMemset(table_dev_.get(), 0, table_bytes));
  free_.reserve(size_t(num_pages));
  for (int page = num_pages - 1; page >= 0; --page) free_.push_back(page);  // the back of the list is page 0
  owned_.assign(size_t(num_slots), {});
  dirty_.assign(size_t(num_slots), false);
}

kernels::KvCacheDesc KvCache::desc() const {
  kernels::KvCacheDesc d;
  d.pool = pool_.as<uint8_t>();
  d.dtype = dtype_;
  d.kv_heads = kv_heads_;
  d.num_pages = num_pages_;
  d.page_bytes = page_bytes_;
  d.layer_stride = layer_stride_;
  d.block_table = table_dev_.as<int>();
  d.max_pages_per_seq = max_pages_per_seq_;
  return d;
}

bool KvCache::ensure(int slot, int tokens) {
  QWEN38_CHECK(slot >= 0 && slot < num_slots_, "KV cache: slot out of range");
  const int need = int(ceil_div(tokens, kernels::kPageTokens));
  QWEN38_CHECK(need <= max_pages_per_seq_, "sequence exceeds the per-sequence context limit (", tokens, " tokens)");
  std::vector<int>& pages = owned_[size_t(slot)];
  const int extra = need - int(pages.size());
  if (extra <= 0) return true;
  if (extra > int(free_.size())) return false;
  int* row = table_host_.as<int>() + size_t(slot) * size_t(max_pages_per_seq_);
  for (int i = 0; i < extra; ++i) {
    row[pages.size()] = free_.back();
    pages.push_back(free_.back());
    free_.pop_back();
  }
  dirty_[size_t(slot)] = true;
  return true;
}

void KvCache::release(int slot) {
  QWEN38_CHECK(slot >= 0 && slot < num_slots_, "KV cache: slot out of range");
  std::vector<int>& pages = owned_[size_t(slot)];
  free_.insert(free_.end(), pages.rbegin(), pages.rend());  // last page first: LIFO reuse
  pages.clear();
}

void KvCache::sync(cudaStream_t stream) {
  for (int s = 0; s < num_slots_; ++s) {
    if (!dirty_[size_t(s)]) continue;
    dirty_[size_t(s)] = false;
    const size_t off = size_t(s) * size_t(max_pages_per_seq_);
    const size_t bytes = owned_[size_t(s)].size() * sizeof(int);
    if (bytes)
      QWEN38_CUDA(cudaMemcpyAsync(table_dev_.as<int>() + off, table_host_.as<int>() + off, bytes,
                                  cudaMemcpyHostToDevice, stream));
  }
}

// ---- GDN state pool ---------------------------------------------------------------------------------
size_t GdnStatePool::bytes_per_slot(const ModelConfig& cfg) {
  const size_t layers = size_t(cfg.num_gdn_layers());
  return layers * size_t(cfg.linear_num_value_heads) * cfg.linear_value_head_dim * cfg.linear_key_head_dim * 4 +
         layers * size_t(cfg.linear_conv_kernel_dim - 1) * size_t(cfg.gdn_conv_dim()) * 2;
}

GdnStatePool::GdnStatePool(const ModelConfig& cfg, int num_slots) : num_gdn_layers_(cfg.num_gdn_layers()) {
  const size_t layers = size_t(num_gdn_layers_);
  recurrent_per_slot_ = layers * size_t(cfg.linear_num_value_heads) * cfg.linear_value_head_dim * cfg.linear_key_head_dim * 4;
  conv_per_slot_ = layers * size_t(cfg.linear_conv_kernel_dim - 1) * size_t(cfg.gdn_conv_dim()) * 2;
  recurrent_ = DeviceBuffer(std::max<size_t>(recurrent_per_slot_ * size_t(num_slots), 256));
  conv_ = DeviceBuffer(std::max<size_t>(conv_per_slot_ * size_t(num_slots), 256));
  QWEN38_CUDA(cudaMemset(recurrent_.get(), 0, recurrent_.bytes()));
  QWEN38_CUDA(cudaMemset(conv_.get(), 0, conv_.bytes()));
}

kernels::GdnStateDesc GdnStatePool::desc() const {
  kernels::GdnStateDesc d;
  d.recurrent = recurrent_.as<float>();
  d.conv = conv_.as<__nv_bfloat16>();
  d.num_gdn_layers = num_gdn_layers_;
  return d;
}

void GdnStatePool::reset(int slot, cudaStream_t stream) {
  if (num_gdn_layers_ == 0) return;
  QWEN38_CUDA(cudaMemsetAsync(recurrent_.as<uint8_t>() + recurrent_per_slot_ * size_t(slot), 0, recurrent_per_slot_, stream));
  QWEN38_CUDA(cudaMemsetAsync(conv_.as<uint8_t>() + conv_per_slot_ * size_t(slot), 0, conv_per_slot_, stream));
}

}  // namespace qwen38
