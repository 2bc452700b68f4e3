// Same include path as the reference's uocr/log.h.  The hot path logs nothing; the macros compile
// to no-ops that still type-check their arguments.
#pragma once
#include <cstdio>
namespace uocr { namespace log {
enum class Level { Trace = 0, Debug = 1, Info = 2, Warn = 3, Error = 4, Off = 5 };
inline void set_level(Level) {}
inline Level level() { return Level::Off; }
inline bool enabled(Level) { return false; }
}}
#define UOCR_LOG(level, ...) do { if (false) std::printf(__VA_ARGS__); } while (0)
#define UOCR_TRACE(...) UOCR_LOG(0, __VA_ARGS__)
#define UOCR_DEBUG(...) UOCR_LOG(1, __VA_ARGS__)
#define UOCR_INFO(...) UOCR_LOG(2, __VA_ARGS__)
#define UOCR_WARN(...) UOCR_LOG(3, __VA_ARGS__)
#define UOCR_ERROR(...) UOCR_LOG(4, __VA_ARGS__)
