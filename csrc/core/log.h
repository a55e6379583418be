// Levelled logging, per-module config logs and the CHK_* early-return macros.
//
// Behavioural model: HCCL's log.h:92-121 (DEBUG/INFO/WARNING/ERROR/RUN_INFO),
// log.h:173-267 (CHK_RET / CHK_PTR_NULL / CHK_PRT_RET) and config_log.h:26
// (module logs gated by HCCL_DEBUG_CONFIG).  Output goes to stderr or to the
// file named by HCCL_LOG_FILE; the level comes from HCCL_LOG_LEVEL
// (debug|info|warning|error|off, default warning).
#pragma once
#include <cstdarg>
#include <cstdint>
#include <string>
#include "hccl/hccl_types.h"

namespace hccl {

enum class LogLevel : int { DEBUG = 0, INFO = 1, WARNING = 2, ERROR = 3, OFF = 4 };
enum LogModule : uint32_t { LOG_MOD_ALG = 1u, LOG_MOD_TASK = 2u, LOG_MOD_RESOURCE = 4u };

LogLevel GetLogLevel();
void SetLogLevel(LogLevel level);
bool ModuleLogEnabled(uint32_t moduleMask);
void SetModuleLogMask(uint32_t mask);  // normally parsed from HCCL_DEBUG_CONFIG
bool EntryLogEnabled();
void SetEntryLogEnabled(bool on);
void LogWrite(LogLevel level, const char* tag, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 5, 6)));
// Structured user-facing input error ("EI0003"-style codes, reference:
// adapter_error_manager_pub.h as used in all_reduce.cc:143-157).
void ReportInputError(const char* code, const char* op, const char* param, const std::string& value,
                      const char* expect);
// Ring of the most recent op records kept for post-mortem (HCCL_DIAGNOSE_ENABLE).
void DiagnoseRecord(const std::string& line);
std::string DiagnoseDump();
const char* ResultString(HcclResult r);

}  // namespace hccl

#define HCCL_LOG_AT(lv, tag, ...)                                                          \
    do {                                                                                   \
        if (static_cast<int>(lv) >= static_cast<int>(::hccl::GetLogLevel()))               \
            ::hccl::LogWrite(lv, tag, __FILE__, __LINE__, __VA_ARGS__);                    \
    } while (0)
#define HCCL_DEBUG(...) HCCL_LOG_AT(::hccl::LogLevel::DEBUG, "DEBUG", __VA_ARGS__)
#define HCCL_INFO(...) HCCL_LOG_AT(::hccl::LogLevel::INFO, "INFO", __VA_ARGS__)
#define HCCL_WARNING(...) HCCL_LOG_AT(::hccl::LogLevel::WARNING, "WARNING", __VA_ARGS__)
#define HCCL_ERROR(...) HCCL_LOG_AT(::hccl::LogLevel::ERROR, "ERROR", __VA_ARGS__)
// Run log: always printed when entry logging is on, independent of the level.
#define HCCL_RUN_INFO(...)                                                                 \
    do {                                                                                   \
        if (::hccl::EntryLogEnabled())                                                     \
            ::hccl::LogWrite(::hccl::LogLevel::OFF, "RUN", __FILE__, __LINE__, __VA_ARGS__); \
    } while (0)
#define HCCL_CONFIG_INFO(moduleMask, ...)                                                  \
    do {                                                                                   \
        if (::hccl::ModuleLogEnabled(moduleMask))                                          \
            ::hccl::LogWrite(::hccl::LogLevel::OFF, "CFG", __FILE__, __LINE__, __VA_ARGS__); \
    } while (0)

#define CHK_RET(expr)                                                                      \
    do {                                                                                   \
        HcclResult _r = (expr);                                                            \
        if (_r != HCCL_SUCCESS) {                                                          \
            HCCL_ERROR("call failed: %s -> %s", #expr, ::hccl::ResultString(_r));          \
            return _r;                                                                     \
        }                                                                                  \
    } while (0)
#define CHK_PTR_NULL(ptr)                                                                  \
    do {                                                                                   \
        if ((ptr) == nullptr) {                                                            \
            HCCL_ERROR("pointer %s is null", #ptr);                                        \
            return HCCL_E_PTR;                                                             \
        }                                                                                  \
    } while (0)
#define CHK_PRT_RET(cond, logstmt, ret)                                                    \
    do {                                                                                   \
        if (cond) {                                                                        \
            logstmt;                                                                       \
            return ret;                                                                    \
        }                                                                                  \
    } while (0)
#define CHK_CUDA(expr)                                                                     \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess) {                                                           \
            HCCL_ERROR("CUDA call failed: %s -> %s", #expr, cudaGetErrorString(_e));       \
            return HCCL_E_RUNTIME;                                                         \
        }                                                                                  \
    } while (0)
