// Calibration text of the performance model: names, parse, canonical format, the shipped B200
// calibration. Format 2 of the reference's text ("key = value" lines, '#' comments; key names as
// in the reference's src/host/perf.cpp:47-116, 715-760): every key required except kernel.* and
// the optional scalars (absent = built-in occupancy / 0).
#pragma once
#include <string>
#include <string_view>

#include "immerdink/immerdink_host.h"
#include "plan.hpp"

namespace imd {

struct CalibError {
  int32_t line = 0;
  int32_t reason = IMD_PERF_CALIB_OK;
  std::string key, message;
};

IMD_INTERNAL const char* perf_class_name(int32_t cls);
IMD_INTERNAL const char* perf_param_name(int32_t cls, int32_t j);
IMD_INTERNAL const char* perf_phase_name(int32_t phase);
IMD_INTERNAL const char* perf_kernel_name(int32_t kernel);
IMD_INTERNAL const char* perf_calib_error_name(int32_t reason);

// Cross-field rules of a calibration (ranges, bands, tie ratio).
IMD_INTERNAL bool perf_calib_valid(const imd_perf_calib_t& c);
// Parses into a full-size struct (struct_size set to sizeof); INVALID_VALUE with *err on failure.
IMD_INTERNAL imd_status_t perf_calib_parse(std::string_view text, imd_perf_calib_t* out,
                                           CalibError* err);
// Canonical text: every key, numbers in the shortest form that parses back to the same double.
IMD_INTERNAL std::string perf_calib_format(const imd_perf_calib_t& c);
// The embedded B200 calibration, parsed once; nullptr (and *err) if its text does not parse.
IMD_INTERNAL const imd_perf_calib_t* perf_calib_shipped(CalibError* err);

}  // namespace imd
