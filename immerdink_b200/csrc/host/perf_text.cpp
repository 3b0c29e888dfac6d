#include "perf_text.hpp"

#include <charconv>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

namespace imd {
namespace {

constexpr int kP = IMD_PERF_MAX_PARAMS;

const char* const kClass[IMD_PERF_CLASS_COUNT] = {"k0", "kf", "kl", "pack", "k4_128x256",
                                                  "k4_128x128", "k4_64x128", "k4_64x64", "k5",
                                                  "direct", "beta", "call"};
const char* const kParam[IMD_PERF_CLASS_COUNT][kP] = {
    {"launch", "byte", "chain", nullptr, nullptr, nullptr},
    {"launch", "byte", "op", "row", "elem", "chain"},
    {"launch", "byte", "op", "l2byte", nullptr, "wave"},
    {"launch", "byte", "op", "dram", "chain", "wave"},
    {"round", "mac1", nullptr, nullptr, "byte", "mac_ktail"},
    {"round", "mac1", "mac2", nullptr, "byte", "mac_ktail"},
    {"round", "mac1", "mac2", nullptr, "byte", "mac_ktail"},
    {"round", "mac1", "mac2", "mac3", "byte", "mac_ktail"},
    {"launch", "byte", "op", "chain", "dram", nullptr},
    {"launch", "byte", "flop", "chain", nullptr, nullptr},
    {"launch", "byte", "chain", nullptr, nullptr, nullptr},
    {"call", "launch", nullptr, nullptr, nullptr, nullptr}};
bool optional_param(int cl, int j) {
  return (cl == IMD_PERF_CLASS_KF && j == 4) || (cl == IMD_PERF_CLASS_PACK && j == 3);
}
const char* const kPhase[IMD_PERF_PHASE_COUNT] = {
    "K0 vec", "KF fused", "KL A", "KL B", "K2 pack A", "K3 pack B", "K4 gemm", "K5 crt",
    "DIRECT", "K5 beta-only", "call", "pack prep", "pack KL"};
const char* const kKernelFixed[IMD_PERF_KERNEL_K5] = {
    "k0", "kf16", "kf4", "kl8", "kl4", "pack", "zero_rows", "direct", "beta", "pack_prep",
    "k4_128x256", "k4_128x128", "k4_64x128", "k4_64x64"};
const char* const kReason[IMD_PERF_CALIB_ERR_COUNT] = {
    "IMD_PERF_CALIB_OK", "IMD_PERF_CALIB_ERR_ARGUMENT", "IMD_PERF_CALIB_ERR_FILE",
    "IMD_PERF_CALIB_ERR_SYNTAX", "IMD_PERF_CALIB_ERR_UNKNOWN_KEY",
    "IMD_PERF_CALIB_ERR_REPEATED_KEY", "IMD_PERF_CALIB_ERR_VALUE", "IMD_PERF_CALIB_ERR_TOO_LONG",
    "IMD_PERF_CALIB_ERR_MISSING_KEY", "IMD_PERF_CALIB_ERR_FORMAT2_KEY",
    "IMD_PERF_CALIB_ERR_INCONSISTENT"};

// Names of the CRT kernels: three row-fastest variants and one batch-fastest per N.
struct CrtNames {
  std::string name[76];
  CrtNames() {
    for (int N = 2; N <= 20; ++N) {
      const int base = 4 * (N - 2);
      const int e[3] = {1, 2, 4};
      for (int v = 0; v < 3; ++v)
        name[base + v] = "k5_n" + std::to_string(N) + "_e" + std::to_string(e[v]);
      name[base + 3] = "k5b_n" + std::to_string(N);
    }
  }
};
const CrtNames& crt_names() {
  static const CrtNames n;
  return n;
}

struct Scalar {
  const char* key;
  double imd_perf_calib_t::*field;
  bool required;
};
const Scalar kScalars[] = {
    {"power.clock_eff_mhz", &imd_perf_calib_t::clock_eff_mhz, true},
    {"power.clock_min_mhz", &imd_perf_calib_t::clock_min_mhz, true},
    {"power.cap_w", &imd_perf_calib_t::power_cap_w, true},
    {"power.idle_w", &imd_perf_calib_t::power_idle_w, true},
    {"power.tc_pj", &imd_perf_calib_t::energy_tc_pj, true},
    {"power.alu_pj", &imd_perf_calib_t::energy_alu_pj, true},
    {"power.byte_pj", &imd_perf_calib_t::energy_byte_pj, true},
    {"power.byte_f_pj", &imd_perf_calib_t::energy_byte_f_pj, false},
    {"power.gamma", &imd_perf_calib_t::energy_gamma, true},
    {"power.act_w", &imd_perf_calib_t::power_act_w, false},
    {"power.act_gap_us", &imd_perf_calib_t::power_act_gap_us, false},
    {"power.dram_pj", &imd_perf_calib_t::energy_dram_pj, false},
    {"power.clock_boost_mhz", &imd_perf_calib_t::clock_boost_mhz, false},
    {"warm.l2_bytes", &imd_perf_calib_t::warm_l2_bytes, true},
    {"warm.l2byte", &imd_perf_calib_t::warm_l2byte_ns, true},
    {"warm.pack_l2_bytes", &imd_perf_calib_t::pack_l2_hit_bytes, false},
    {"warm.pack_l2_planes", &imd_perf_calib_t::pack_l2_planes, false},
    {"warm.call_ns", &imd_perf_calib_t::warm_call_ns, false},
    {"warm.clean_byte", &imd_perf_calib_t::warm_clean_byte_ns, false},
    {"rank.tie_ratio", &imd_perf_calib_t::tie_ratio, true}};
const Scalar kPeaks[] = {
    {"peak_dram_bytes_per_s", &imd_perf_calib_t::peak_dram_bytes_per_s, true},
    {"peak_int8_ops_per_s", &imd_perf_calib_t::peak_int8_ops_per_s, true},
    {"peak_fp64_flops_per_s", &imd_perf_calib_t::peak_fp64_flops_per_s, true},
    {"l2_bytes", &imd_perf_calib_t::l2_bytes, true}};
const char* const kBandCall[3] = {"band.call_small", "band.call_mid", "band.call_large"};
constexpr const char* kKlDrop = "warm.kl_drop";

struct Text {
  const char* key;
  size_t offset, capacity;
};
const Text kTexts[] = {{"gpu", offsetof(imd_perf_calib_t, gpu), 64},
                       {"date", offsetof(imd_perf_calib_t, date), 32},
                       {"version", offsetof(imd_perf_calib_t, version), 64},
                       {"clocks", offsetof(imd_perf_calib_t, clocks), 128},
                       {"notes", offsetof(imd_perf_calib_t, notes), 128}};

std::string_view trim(std::string_view s) {
  while (!s.empty() && (s.front() == ' ' || s.front() == '\t' || s.front() == '\r')) s.remove_prefix(1);
  while (!s.empty() && (s.back() == ' ' || s.back() == '\t' || s.back() == '\r')) s.remove_suffix(1);
  return s;
}

// Whitespace-separated finite numbers; exactly `want` of them.
bool numbers(std::string_view v, double* out, int want) {
  int got = 0;
  while (true) {
    v = trim(v);
    if (v.empty()) break;
    size_t end = 0;
    while (end < v.size() && v[end] != ' ' && v[end] != '\t') ++end;
    double x = 0;
    const std::string tok(v.substr(0, end));
    char* stop = nullptr;
    x = std::strtod(tok.c_str(), &stop);
    if (stop == tok.c_str() || *stop != '\0' || !std::isfinite(x)) return false;
    if (got < want) out[got] = x;
    ++got;
    v.remove_prefix(end);
  }
  return got == want;
}

imd_perf_kernel_t builtin_kernel() { return imd_perf_kernel_t{1, 0, 0, 256}; }

imd_status_t fail(CalibError* e, int32_t line, int32_t reason, std::string_view key,
                  const std::string& what) {
  if (e != nullptr) {
    e->line = line, e->reason = reason;
    e->key = std::string(key.substr(0, 63));
    e->message = (line > 0 ? "line " + std::to_string(line) + ": " : std::string()) +
                 (key.empty() ? std::string() : e->key + ": ") + what;
    if (e->message.size() > 191) e->message.resize(191);
  }
  return IMD_STATUS_INVALID_VALUE;
}

void append_number(std::string* s, double v) {
  char buf[40];
  const auto r = std::to_chars(buf, buf + sizeof buf, v);  // shortest round-trip form
  s->append(buf, r.ptr);
}

#include "perf_calib_b200.inc"

}  // namespace

const char* perf_class_name(int32_t cls) {
  return cls >= 0 && cls < IMD_PERF_CLASS_COUNT ? kClass[cls] : nullptr;
}
const char* perf_param_name(int32_t cls, int32_t j) {
  return cls >= 0 && cls < IMD_PERF_CLASS_COUNT && j >= 0 && j < kP ? kParam[cls][j] : nullptr;
}
const char* perf_phase_name(int32_t phase) {
  return phase >= 0 && phase < IMD_PERF_PHASE_COUNT ? kPhase[phase] : nullptr;
}
const char* perf_kernel_name(int32_t k) {
  if (k < 0 || k >= IMD_PERF_KERNEL_COUNT) return nullptr;
  return k < IMD_PERF_KERNEL_K5 ? kKernelFixed[k] : crt_names().name[k - IMD_PERF_KERNEL_K5].c_str();
}
const char* perf_calib_error_name(int32_t reason) {
  return reason >= 0 && reason < IMD_PERF_CALIB_ERR_COUNT ? kReason[reason] : nullptr;
}

bool perf_calib_valid(const imd_perf_calib_t& c) {
  const auto nonneg = [](double v) { return std::isfinite(v) && v >= 0; };
  if (c.format != 2 || c.sm_count < 1) return false;
  for (const Scalar& s : kPeaks)
    if (!(c.*(s.field) > 0) || !std::isfinite(c.*(s.field))) return false;
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl)
    for (int j = 0; j < kP; ++j) {
      const double v = c.param[cl * kP + j];
      if (!std::isfinite(v) || (cl != IMD_PERF_CLASS_CALL && v < 0)) return false;
    }
  const double drop = c.param[IMD_PERF_PARAM_KL_DROP_SLOT];
  if (!(drop >= 0 && drop <= 1)) return false;
  for (int k = 0; k < IMD_PERF_KERNEL_COUNT; ++k) {
    const imd_perf_kernel_t& q = c.kernel[k];
    if (q.resident < 1 || q.regs < 0 || q.smem_bytes < 0 || q.threads < 0) return false;
  }
  for (const Scalar& s : kScalars)
    if (!nonneg(c.*(s.field))) return false;
  if (c.pack_l2_planes != 0 && c.pack_l2_planes != 1) return false;
  if (c.clock_boost_mhz > 0 && !(c.clock_boost_mhz >= c.clock_eff_mhz)) return false;
  if (c.power_cap_w > 0 &&
      !(c.clock_eff_mhz > 0 && c.clock_min_mhz > 0 && c.clock_min_mhz <= c.clock_eff_mhz))
    return false;
  if (!(c.tie_ratio >= 1 && c.tie_ratio <= 1.25)) return false;
  const auto band_ok = [](const double* b) {
    return std::isfinite(b[0]) && std::isfinite(b[1]) && b[0] > 0 && b[0] <= b[1];
  };
  for (const auto& b : c.band_call)
    if (!band_ok(b)) return false;
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl)
    if (!band_ok(c.band_class[cl])) return false;
  return true;
}

imd_status_t perf_calib_parse(std::string_view text, imd_perf_calib_t* out, CalibError* err) {
  imd_perf_calib_t c;
  std::memset(&c, 0, sizeof c);
  c.struct_size = sizeof c;
  for (int k = 0; k < IMD_PERF_KERNEL_COUNT; ++k) c.kernel[k] = builtin_kernel();
  std::map<std::string, int, std::less<>> seen;  // key -> line
  // every key this format knows -> how to store it
  enum Kind { kFormat, kSm, kTextKey, kPeak, kParamKey, kScalar, kBandCallKey, kBandClass, kKernel, kDrop };
  struct Slot {
    Kind kind;
    int a = 0, b = 0;
    bool required = true;
  };
  std::map<std::string, Slot, std::less<>> keys;
  keys["format"] = {kFormat};
  keys["sm_count"] = {kSm};
  for (int i = 0; i < 5; ++i) keys[kTexts[i].key] = {kTextKey, i};
  for (int i = 0; i < 4; ++i) keys[kPeaks[i].key] = {kPeak, i};
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl)
    for (int j = 0; j < kP; ++j)
      if (kParam[cl][j] != nullptr)
        keys[std::string(kClass[cl]) + "." + kParam[cl][j]] = {kParamKey, cl, j, !optional_param(cl, j)};
  for (size_t i = 0; i < sizeof kScalars / sizeof kScalars[0]; ++i)
    keys[kScalars[i].key] = {kScalar, static_cast<int>(i), 0, kScalars[i].required};
  for (int i = 0; i < 3; ++i) keys[kBandCall[i]] = {kBandCallKey, i};
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl) keys[std::string("band.") + kClass[cl]] = {kBandClass, cl};
  for (int k = 0; k < IMD_PERF_KERNEL_COUNT; ++k)
    keys[std::string("kernel.") + perf_kernel_name(k)] = {kKernel, k, 0, false};
  keys[kKlDrop] = {kDrop, 0, 0, false};
  for (const char* retired : {"kf.op_eps", "kl.op_eps", "pack.op_eps"})
    keys[retired] = {kDrop, 1, 0, false};  // accepted and discarded

  int32_t line_no = 0;
  size_t pos = 0;
  while (pos <= text.size()) {
    const size_t nl = text.find('\n', pos);
    std::string_view line = text.substr(pos, nl == std::string_view::npos ? text.size() - pos : nl - pos);
    pos = nl == std::string_view::npos ? text.size() + 1 : nl + 1;
    ++line_no;
    line = trim(line);
    if (line.empty() || line.front() == '#') continue;
    const size_t eq = line.find('=');
    if (eq == std::string_view::npos)
      return fail(err, line_no, IMD_PERF_CALIB_ERR_SYNTAX, "", "not blank, a '#' comment or key = value");
    const std::string_view key = trim(line.substr(0, eq)), value = trim(line.substr(eq + 1));
    const auto it = keys.find(key);
    if (key.empty() || it == keys.end())
      return fail(err, line_no, IMD_PERF_CALIB_ERR_UNKNOWN_KEY, key, "unknown key");
    if (const auto s = seen.find(key); s != seen.end())
      return fail(err, line_no, IMD_PERF_CALIB_ERR_REPEATED_KEY, key,
                  "already given on line " + std::to_string(s->second));
    seen.emplace(std::string(key), line_no);
    const Slot& sl = it->second;
    double v[4] = {0, 0, 0, 0};
    const auto bad = [&](const char* what) {
      return fail(err, line_no, IMD_PERF_CALIB_ERR_VALUE, key, what);
    };
    switch (sl.kind) {
      case kFormat:
        if (!numbers(value, v, 1) || v[0] != 2) return bad("this engine reads format 2 only");
        c.format = 2;
        break;
      case kSm:
        if (!numbers(value, v, 1) || v[0] < 1 || v[0] > 1e6 || v[0] != std::floor(v[0]))
          return bad("a positive integer is needed");
        c.sm_count = static_cast<int32_t>(v[0]);
        break;
      case kTextKey: {
        const Text& t = kTexts[sl.a];
        if (value.size() + 1 > t.capacity)
          return fail(err, line_no, IMD_PERF_CALIB_ERR_TOO_LONG, key,
                      "value is " + std::to_string(value.size()) + " bytes, the field holds " +
                          std::to_string(t.capacity - 1));
        std::memcpy(reinterpret_cast<char*>(&c) + t.offset, value.data(), value.size());
        break;
      }
      case kPeak:
        if (!numbers(value, v, 1) || !(v[0] > 0)) return bad("a positive number is needed");
        c.*(kPeaks[sl.a].field) = v[0];
        break;
      case kParamKey:
        if (!numbers(value, v, 1) || (sl.a != IMD_PERF_CLASS_CALL && v[0] < 0))
          return bad("a number >= 0 is needed");
        c.param[sl.a * kP + sl.b] = v[0];
        break;
      case kScalar:
        if (!numbers(value, v, 1) || v[0] < 0) return bad("a number >= 0 is needed");
        c.*(kScalars[sl.a].field) = v[0];
        break;
      case kBandCallKey:
      case kBandClass: {
        if (!numbers(value, v, 2) || !(v[0] > 0 && v[0] <= v[1])) return bad("lo hi with 0 < lo <= hi");
        double* b = sl.kind == kBandCallKey ? c.band_call[sl.a] : c.band_class[sl.a];
        b[0] = v[0], b[1] = v[1];
        break;
      }
      case kKernel:
        if (!numbers(value, v, 4) || v[0] < 1 || v[1] < 0 || v[2] < 0 || v[3] < 0)
          return bad("resident >= 1, registers, shared bytes, threads");
        c.kernel[sl.a] = imd_perf_kernel_t{static_cast<int32_t>(v[0]), static_cast<int32_t>(v[1]),
                                           static_cast<int32_t>(v[2]), static_cast<int32_t>(v[3])};
        break;
      case kDrop:
        if (!numbers(value, v, 1) || v[0] < 0 || (sl.a == 0 && v[0] > 1)) return bad("out of range");
        if (sl.a == 0) c.param[IMD_PERF_PARAM_KL_DROP_SLOT] = v[0];
        break;
    }
  }
  // missing keys, in a fixed order: scalars first, then the parameters, then the bands
  std::vector<std::string> order = {"format", "gpu", "sm_count", "date", "version", "clocks", "notes"};
  for (const Scalar& s : kPeaks) order.push_back(s.key);
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl)
    for (int j = 0; j < kP; ++j)
      if (kParam[cl][j] != nullptr && !optional_param(cl, j))
        order.push_back(std::string(kClass[cl]) + "." + kParam[cl][j]);
  for (const Scalar& s : kScalars)
    if (s.required) order.push_back(s.key);
  for (const char* k : kBandCall) order.push_back(k);
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl) order.push_back(std::string("band.") + kClass[cl]);
  for (const std::string& k : order)
    if (seen.find(k) == seen.end())
      return fail(err, 0, IMD_PERF_CALIB_ERR_MISSING_KEY, k, "missing key");
  if (!perf_calib_valid(c))
    return fail(err, 0, IMD_PERF_CALIB_ERR_INCONSISTENT, "",
                "a cross-key rule is broken (power clocks, rank.tie_ratio in [1, 1.25], bands)");
  *out = c;
  if (err != nullptr) *err = CalibError{};
  return IMD_STATUS_SUCCESS;
}

std::string perf_calib_format(const imd_perf_calib_t& c) {
  std::string s = "# immerdink performance-model calibration, format 2 (this engine's kernels).\n"
                  "# Parameters: <class>.<feature> = ns per feature unit.\n";
  const auto text = [&](const char* key, const char* v) { s += std::string(key) + " = " + v + "\n"; };
  const auto num = [&](const std::string& key, double v) {
    s += key + " = ";
    append_number(&s, v);
    s += "\n";
  };
  s += "format = 2\n";
  text("gpu", c.gpu);
  s += "sm_count = " + std::to_string(c.sm_count) + "\n";
  text("date", c.date);
  text("version", c.version);
  text("clocks", c.clocks);
  text("notes", c.notes);
  for (const Scalar& k : kPeaks) num(k.key, c.*(k.field));
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl)
    for (int j = 0; j < kP; ++j) {
      if (kParam[cl][j] == nullptr) continue;
      const double v = c.param[cl * kP + j];
      if (optional_param(cl, j) && v == 0) continue;
      num(std::string(kClass[cl]) + "." + kParam[cl][j], v);
    }
  s += "# Occupancy: kernel.<name> = CTAs per SM, registers per thread, shared bytes, threads per CTA.\n";
  for (int k = 0; k < IMD_PERF_KERNEL_COUNT; ++k) {
    const imd_perf_kernel_t& q = c.kernel[k];
    s += std::string("kernel.") + perf_kernel_name(k) + " = " + std::to_string(q.resident) + " " +
         std::to_string(q.regs) + " " + std::to_string(q.smem_bytes) + " " + std::to_string(q.threads) + "\n";
  }
  for (const Scalar& k : kScalars) {
    const double v = c.*(k.field);
    if (!k.required && v == 0) continue;
    num(k.key, v);
  }
  if (c.param[IMD_PERF_PARAM_KL_DROP_SLOT] != 0) num(kKlDrop, c.param[IMD_PERF_PARAM_KL_DROP_SLOT]);
  const auto band = [&](const std::string& key, const double* b) {
    s += key + " = ";
    append_number(&s, b[0]);
    s += " ";
    append_number(&s, b[1]);
    s += "\n";
  };
  for (int i = 0; i < 3; ++i) band(kBandCall[i], c.band_call[i]);
  for (int cl = 0; cl < IMD_PERF_CLASS_COUNT; ++cl) band(std::string("band.") + kClass[cl], c.band_class[cl]);
  return s;
}

const imd_perf_calib_t* perf_calib_shipped(CalibError* err) {
  static std::once_flag once;
  static imd_perf_calib_t cal;
  static CalibError why;
  static bool ok = false;
  std::call_once(once, [] { ok = perf_calib_parse(kShippedCalibration, &cal, &why) == IMD_STATUS_SUCCESS; });
  if (!ok && err != nullptr) {
    *err = why;
    err->message = "shipped calibration: " + why.message;
    if (err->message.size() > 191) err->message.resize(191);
  }
  return ok ? &cal : nullptr;
}

}  // namespace imd
