// GEMM tile-configuration table: (bits, n, k, m_max) -> config id, stored as JSON and installed into the
// kernel library's dispatcher through its lookup hook (reference src/tuning.cpp, include/qwen38/tuning.h).
#include <algorithm>
#include <fstream>
#include <iterator>

#include "json_min.h"
#include "qwen38/api.h"

namespace qwen38 {

namespace {
std::vector<TuningEntry> g_table;
int table_lookup(int bits, int n, int k, int m) { return lookup_tuning(bits, n, k, m); }
}  // namespace

void install_tuning(std::vector<TuningEntry> entries) {
  std::sort(entries.begin(), entries.end(), [](const TuningEntry& a, const TuningEntry& b) { return a.m_max < b.m_max; });
  g_table = std::move(entries);
  kernels::set_qgemm_tuning(g_table.empty() ? nullptr : &table_lookup);
}

int lookup_tuning(int bits, int n, int k, int m) {
  for (const TuningEntry& e : g_table)  // sorted by m_max: the smallest matching ceiling wins
    if (e.bits == bits && e.n == n && e.k == k && m <= e.m_max) return e.config;
  return kernels::kGemmConfigAuto;
}

void load_tuning(const std::string& path) {
  std::ifstream in(path);
  QWEN38_CHECK(in.good(), "cannot open tuning table ", path);
  const std::string text((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  std::vector<TuningEntry> entries;
  try {
    const jsonmin::Value j = jsonmin::parse(text);
    for (const auto& e : j.at("entries").arr) {
      TuningEntry t;
      t.bits = int(e.at("bits").as_int());
      t.n = int(e.at("n").as_int());
      t.k = int(e.at("k").as_int());
      t.m_max = int(e.at("m_max").as_int());
      t.config = int(e.at("config").as_int());
      t.us = e.has("us") ? e.at("us").as_double() : 0.0;
      entries.push_back(t);
    }
  } catch (const std::exception& e) {
    fail(path + ": malformed tuning table: " + e.what());
  }
  install_tuning(std::move(entries));
}

void save_tuning(const std::string& path, const std::vector<TuningEntry>& entries, const std::string& device) {
  std::ofstream out(path);
  QWEN38_CHECK(out.good(), "cannot write ", path);
  out << "{\n \"device\": \"" << device << "\",\n \"entries\": [\n";
  for (size_t i = 0; i < entries.size(); ++i) {
    const TuningEntry& e = entries[i];
    out << "  {\"bits\": " << e.bits << ", \"n\": " << e.n << ", \"k\": " << e.k << ", \"m_max\": " << e.m_max
        << ", \"config\": " << e.config << ", \"us\": " << e.us << "}" << (i + 1 < entries.size() ? "," : "") << "\n";
  }
  out << " ]\n}\n";
}

}  // namespace qwen38
