// Host-only pieces: error helpers, 16-bit float conversions, ModelConfig, the .q38 reader and the BQ
// spec decoder. Behaviour follows the reference's src/model_file.cpp and src/bq_host.cpp (same checks,
// same error conditions); the file format is the reference's docs/FORMAT.md.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <fstream>

#include "json_min.h"
#include "qwen38/api.h"

namespace qwen38 {

void fail(const std::string& message) { throw Error(message); }

void throw_kernel_error(const char* message) { throw Error(std::string("kernel launcher: ") + message); }

std::string format_check_failure(const char* expr, const char* file, int line, const std::string& msg) {
  std::string s = std::string(file) + ":" + std::to_string(line) + ": check failed: " + expr;
  return msg.empty() ? s : s + ": " + msg;
}

uint16_t f32_to_bf16(float f) {
  const uint32_t u = std::bit_cast<uint32_t>(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40u);
  return uint16_t((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

float f16_to_f32(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
  if (e == 0) {
    const float v = std::ldexp(float(m), -24);
    return sign ? -v : v;
  }
  if (e == 31) return std::bit_cast<float>(sign | 0x7f800000u | (m << 13));
  return std::bit_cast<float>(sign | ((e + 112u) << 23) | (m << 13));
}

uint16_t f32_to_f16(float f) {
  const uint32_t u = std::bit_cast<uint32_t>(f);
  const uint32_t sign = (u >> 16) & 0x8000u, mag = u & 0x7fffffffu;
  if (mag > 0x7f800000u) return uint16_t(sign | 0x7e00u);
  if (mag >= 0x477ff000u) return uint16_t(sign | 0x7c00u);
  if (mag < 0x38800000u) return uint16_t(sign | uint32_t(std::nearbyint(std::bit_cast<float>(mag) * 16777216.0f)));
  return uint16_t(sign | (((mag + 0xfffu + ((mag >> 13) & 1u)) >> 13) - (112u << 10)));
}

// ---- ModelConfig ------------------------------------------------------------------------------------
int ModelConfig::num_attention_layers() const {
  int n = 0;
  for (uint8_t a : is_attention) n += a != 0;
  return n;
}
int ModelConfig::num_gdn_layers() const { return num_layers - num_attention_layers(); }
int ModelConfig::attn_index(int layer) const {
  if (!is_attention[size_t(layer)]) return -1;
  int idx = 0;
  for (int i = 0; i < layer; ++i) idx += is_attention[size_t(i)] != 0;
  return idx;
}
int ModelConfig::gdn_index(int layer) const {
  if (is_attention[size_t(layer)]) return -1;
  int idx = 0;
  for (int i = 0; i < layer; ++i) idx += is_attention[size_t(i)] == 0;
  return idx;
}

void ModelConfig::validate() const {
  QWEN38_CHECK(num_layers > 0 && int(is_attention.size()) == num_layers, "layer_types size");
  QWEN38_CHECK(hidden_size > 0 && hidden_size % 128 == 0, "hidden_size must be a multiple of 128, got ", hidden_size);
  QWEN38_CHECK(vocab_size > 0 && vocab_size % 128 == 0, "vocab_size must be a multiple of 128, got ", vocab_size);
  QWEN38_CHECK(intermediate_size > 0 && intermediate_size % 64 == 0, "intermediate_size must be a multiple of 64");
  if (num_attention_layers() > 0) {
    QWEN38_CHECK(head_dim == 256, "attention kernels implement head_dim 256, got ", head_dim);
    QWEN38_CHECK(rotary_dim == 64, "RoPE kernel implements rotary_dim 64, got ", rotary_dim);
    QWEN38_CHECK(num_key_value_heads > 0 && num_attention_heads % num_key_value_heads == 0, "GQA heads");
    QWEN38_CHECK(attn_group() <= 8, "GQA group > 8 is not implemented");
    QWEN38_CHECK(num_attention_heads + 2 * num_key_value_heads <= 32, "more than 32 q + k + v heads per token");
  }
  if (num_gdn_layers() > 0) {
    QWEN38_CHECK(linear_key_head_dim == 128 && linear_value_head_dim == 128, "GDN kernels implement 128-dim heads");
    QWEN38_CHECK(linear_conv_kernel_dim == 4, "GDN conv kernel implements width 4");
    QWEN38_CHECK(linear_num_key_heads > 0 && linear_num_value_heads % linear_num_key_heads == 0, "GDN head ratio");
  }
  QWEN38_CHECK(norm_folded, "model files without folded norms are not supported");
}

std::string ModelConfig::summary() const {
  std::ostringstream os;
  os << "hidden " << hidden_size << ", layers " << num_layers << " (" << num_attention_layers() << " attention / "
     << num_gdn_layers() << " GDN), vocab " << vocab_size << ", ffn " << intermediate_size << ", attn "
     << num_attention_heads << "q/" << num_key_value_heads << "kv x" << head_dim << ", gdn " << linear_num_key_heads
     << "k/" << linear_num_value_heads << "v x" << linear_key_head_dim;
  return os.str();
}

// ---- model file -----------------------------------------------------------------------------------
const char* dtype_name(DType dtype) {
  constexpr const char* kNames[] = {"bq4", "bq5", "bq6", "bq8", "bf16", "f32"};
  return kNames[int(dtype)];
}

namespace {

DType dtype_from(const std::string& s) {
  for (int i = 0; i < 6; ++i)
    if (s == dtype_name(DType(i))) return DType(i);
  fail("unknown dtype " + s);
}

ModelConfig read_config(const jsonmin::Value& j) {
  ModelConfig c;
  auto geti = [&](const char* key) { return int(j.at(key).as_int()); };
  c.hidden_size = geti("hidden_size");
  c.num_layers = geti("num_layers");
  c.vocab_size = geti("vocab_size");
  c.intermediate_size = geti("intermediate_size");
  c.num_attention_heads = geti("num_attention_heads");
  c.num_key_value_heads = geti("num_key_value_heads");
  c.head_dim = geti("head_dim");
  c.rotary_dim = geti("rotary_dim");
  c.rope_theta = j.at("rope_theta").as_double();
  c.linear_num_key_heads = geti("linear_num_key_heads");
  c.linear_num_value_heads = geti("linear_num_value_heads");
  c.linear_key_head_dim = geti("linear_key_head_dim");
  c.linear_value_head_dim = geti("linear_value_head_dim");
  c.linear_conv_kernel_dim = geti("linear_conv_kernel_dim");
  c.rms_norm_eps = float(j.at("rms_norm_eps").as_double());
  c.max_position_embeddings = geti("max_position_embeddings");
  c.norm_folded = j.has("norm_folded") && j.at("norm_folded").as_bool();
  for (const auto& t : j.at("layer_types").arr) {
    const std::string& kind = t.as_string();
    QWEN38_CHECK(kind == "full_attention" || kind == "linear_attention", "layer type ", kind);
    c.is_attention.push_back(kind == "full_attention" ? 1 : 0);
  }
  if (j.has("eos_token_ids"))
    for (const auto& e : j.at("eos_token_ids").arr) c.eos_token_ids.push_back(int32_t(e.as_int()));
  return c;
}

}  // namespace

int64_t TensorInfo::numel() const {
  int64_t n = 1;
  for (int64_t d : shape) n *= d;
  return n;
}

std::unique_ptr<ModelFile> ModelFile::open(const std::string& path) {
  std::unique_ptr<ModelFile> mf(new ModelFile());
  mf->path_ = path;
  {
    std::ifstream in(path, std::ios::binary);
    QWEN38_CHECK(in.good(), "cannot open ", path);
    char magic[8] = {};
    in.read(magic, 8);
    QWEN38_CHECK(in.good() && std::memcmp(magic, "QW38MDL1", 8) == 0, path, " is not a .q38 model file");
    uint64_t header_len = 0;
    in.read(reinterpret_cast<char*>(&header_len), 8);
    QWEN38_CHECK(in.good() && header_len > 0 && header_len < (1ull << 30), "bad header length");
    mf->header_.resize(header_len);
    in.read(mf->header_.data(), std::streamsize(header_len));
    QWEN38_CHECK(in.good(), "truncated header");
    in.seekg(0, std::ios::end);
    mf->file_size_ = uint64_t(in.tellg());
    mf->data_start_ = uint64_t(align_up(int64_t(16 + header_len), 4096));
  }
  jsonmin::Value j;
  try {
    j = jsonmin::parse(mf->header_);
    QWEN38_CHECK(j.at("format").as_string() == "qwen38-model", "not a qwen38 model header");
    QWEN38_CHECK(j.at("format_version").as_int() == 1, "unsupported format_version");
    mf->config_ = read_config(j.at("config"));
    if (j.has("recipe") && j.at("recipe").has("name")) mf->recipe_ = j.at("recipe").at("name").as_string();
    for (const auto& [name, rec] : j.at("tensors").obj) {
      TensorInfo t;
      t.name = name;
      t.dtype = dtype_from(rec.at("dtype").as_string());
      for (const auto& d : rec.at("shape").arr) t.shape.push_back(d.as_int());
      t.rows = rec.has("rows") ? rec.at("rows").as_int() : (t.shape.empty() ? 1 : t.shape[0]);
      if (is_bq(t.dtype)) {
        QWEN38_CHECK(t.shape.size() == 2, name, ": BQ tensors are rank 2");
        QWEN38_CHECK(rec.has("group_size") && rec.at("group_size").as_int() == 64, name, ": group_size must be 64");
        QWEN38_CHECK(t.shape[0] % 128 == 0 && t.shape[1] % 64 == 0, name, ": BQ shape constraints");
        const auto& planes = rec.at("planes");
        t.lo_offset = planes.at("lo").arr.at(0).as_int();
        t.lo_bytes = planes.at("lo").arr.at(1).as_int();
        if (planes.has("hi")) {
          t.hi_offset = planes.at("hi").arr.at(0).as_int();
          t.hi_bytes = planes.at("hi").arr.at(1).as_int();
        }
        t.sc_offset = planes.at("scales").arr.at(0).as_int();
        t.sc_bytes = planes.at("scales").arr.at(1).as_int();
        const int64_t nk = t.shape[0] * t.shape[1];
        QWEN38_CHECK(t.lo_bytes == nk / 2, name, ": lo plane size");
        QWEN38_CHECK(t.hi_bytes == nk * (bq_bits(t.dtype) - 4) / 8, name, ": hi plane size");
        QWEN38_CHECK(t.sc_bytes == t.shape[0] * (t.shape[1] / 64) * 2, name, ": scale plane size");
      } else {
        t.offset = rec.at("offset").as_int();
        t.bytes = rec.at("bytes").as_int();
        QWEN38_CHECK(t.bytes == t.numel() * (t.dtype == DType::BF16 ? 2 : 4), name, ": size mismatch");
      }
      mf->tensors_.emplace(name, std::move(t));
    }
    if (j.has("resources"))
      for (const auto& [name, rec] : j.at("resources").obj)
        mf->resources_[name] = {rec.at("offset").as_int(), rec.at("bytes").as_int()};
  } catch (const Error&) {
    throw;
  } catch (const std::exception& e) {
    fail(path + ": malformed header: " + e.what());
  }

  mf->fd_ = ::open(path.c_str(), O_RDONLY);
  QWEN38_CHECK(mf->fd_ >= 0, "cannot open ", path);
  void* p = ::mmap(nullptr, mf->file_size_, PROT_READ, MAP_PRIVATE, mf->fd_, 0);
  QWEN38_CHECK(p != MAP_FAILED, "mmap failed for ", path);
  mf->base_ = static_cast<const uint8_t*>(p);
  mf->mapped_size_ = mf->file_size_;

  // every object must lie inside the file (catches truncated copies)
  for (const auto& [name, t] : mf->tensors_) {
    auto inside = [&](int64_t off, int64_t size) {
      QWEN38_CHECK(off >= 0 && size >= 0 && mf->data_start_ + uint64_t(off + size) <= mf->file_size_, name,
                   ": object outside the file (truncated download?)");
    };
    if (is_bq(t.dtype)) {
      inside(t.lo_offset, t.lo_bytes);
      inside(t.hi_offset, t.hi_bytes);
      inside(t.sc_offset, t.sc_bytes);
    } else {
      inside(t.offset, t.bytes);
    }
  }
  mf->config_.validate();
  return mf;
}

ModelFile::~ModelFile() {
  if (base_ && mapped_size_) ::munmap(const_cast<uint8_t*>(base_), mapped_size_);
  if (fd_ >= 0) ::close(fd_);
}

const TensorInfo& ModelFile::tensor(const std::string& name) const {
  const auto it = tensors_.find(name);
  QWEN38_CHECK(it != tensors_.end(), "tensor '", name, "' not found in ", path_);
  return it->second;
}

std::span<const uint8_t> ModelFile::data(int64_t offset, int64_t size) const {
  QWEN38_CHECK(offset >= 0 && size >= 0 && data_start_ + uint64_t(offset + size) <= file_size_, "data range");
  return {base_ + data_start_ + offset, size_t(size)};
}

std::span<const uint8_t> ModelFile::resource(const std::string& name) const {
  const auto it = resources_.find(name);
  if (it == resources_.end()) return {};
  return data(it->second.first, it->second.second);
}

int64_t ModelFile::total_weight_bytes() const {
  int64_t total = 0;
  for (const auto& [name, t] : tensors_) total += t.storage_bytes();
  return total;
}

// ---- BQ spec decoder (docs/FORMAT.md 2.2-2.5) -------------------------------------------------------
BQView BQView::from_file(const ModelFile& file, const std::string& name) {
  const TensorInfo& t = file.tensor(name);
  QWEN38_CHECK(is_bq(t.dtype), name, " is not a BQ tensor");
  BQView v;
  v.bits = bq_bits(t.dtype);
  v.n = t.shape[0];
  v.k = t.shape[1];
  v.rows = t.rows;
  v.lo = file.data(t.lo_offset, t.lo_bytes).data();
  v.hi = t.hi_bytes ? file.data(t.hi_offset, t.hi_bytes).data() : nullptr;
  v.scales = reinterpret_cast<const uint16_t*>(file.data(t.sc_offset, t.sc_bytes).data());
  return v;
}

namespace {
inline uint32_t word_at(const uint8_t* p) {
  uint32_t v;
  std::memcpy(&v, p, 4);
  return v;
}
}  // namespace

int BQView::code(int64_t row, int64_t col) const {
  const int nl = int(row & 63), kl = int(col & 15);
  const int64_t slab = (row >> 6) * (k >> 4) + (col >> 4);
  const int lane = 4 * (nl & 7) + ((kl & 7) >> 1), pair = 2 * (nl >> 3) + (kl >> 3), half = (kl & 1) ? 16 : 0;
  auto nib = [&](const uint8_t* plane) {
    return (word_at(plane + slab * 512 + lane * 16 + 4 * (pair >> 2)) >> (half + 4 * (pair & 3))) & 15u;
  };
  unsigned u = nib(lo);
  if (bits == 5) u |= ((word_at(hi + slab * 128 + lane * 4) >> (half + pair)) & 1u) << 4;
  else if (bits == 6) u |= ((word_at(hi + slab * 256 + lane * 8 + 4 * (pair >> 3)) >> (half + 2 * (pair & 7))) & 3u) << 4;
  else if (bits == 8) u |= nib(hi) << 4;
  return int(u) - (1 << (bits - 1));
}

uint16_t BQView::scale_bits(int64_t row, int64_t group) const {
  const int nl = int(row & 63);
  return scales[((row >> 6) * (k >> 6) + group) * 64 + (nl & 7) * 8 + (nl >> 3)];
}

float BQView::scale(int64_t row, int64_t group) const { return bf16_to_f32(scale_bits(row, group)); }
float BQView::weight(int64_t row, int64_t col) const { return round_bf16(float(code(row, col)) * scale(row, col >> 6)); }
void BQView::dequant_row(int64_t row, float* out) const {
  for (int64_t c = 0; c < k; ++c) out[c] = weight(row, c);
}
std::vector<float> BQView::dequant_all() const {
  std::vector<float> w(size_t(n * k));
  for (int64_t r = 0; r < n; ++r) dequant_row(r, w.data() + r * k);
  return w;
}

}  // namespace qwen38
