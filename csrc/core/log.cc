#include "log.h"
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <unistd.h>

namespace hccl {
namespace {
struct LogState {
    LogLevel level = LogLevel::WARNING;
    uint32_t moduleMask = 0;
    bool entryLog = false;
    FILE* out = stderr;
    std::mutex mu;
    std::deque<std::string> diag;
    size_t diagCap = 2000;  // HCCL keeps the last 2000 ops (HCCL_DIAGNOSE_ENABLE.md)
    LogState()
    {
        if (const char* lv = getenv("HCCL_LOG_LEVEL")) {
            if (!strcasecmp(lv, "debug") || !strcmp(lv, "0")) level = LogLevel::DEBUG;
            else if (!strcasecmp(lv, "info") || !strcmp(lv, "1")) level = LogLevel::INFO;
            else if (!strcasecmp(lv, "warning") || !strcmp(lv, "2")) level = LogLevel::WARNING;
            else if (!strcasecmp(lv, "error") || !strcmp(lv, "3")) level = LogLevel::ERROR;
            else if (!strcasecmp(lv, "off") || !strcmp(lv, "4")) level = LogLevel::OFF;
        }
        if (const char* f = getenv("HCCL_LOG_FILE")) {
            if (FILE* fp = fopen(f, "a")) out = fp;
        }
        if (const char* e = getenv("HCCL_ENTRY_LOG_ENABLE")) entryLog = (strcmp(e, "1") == 0);
    }
};
LogState& S()
{
    static LogState s;
    return s;
}
}  // namespace

LogLevel GetLogLevel() { return S().level; }
void SetLogLevel(LogLevel level) { S().level = level; }
bool ModuleLogEnabled(uint32_t m) { return (S().moduleMask & m) != 0; }
void SetModuleLogMask(uint32_t mask) { S().moduleMask = mask; }
bool EntryLogEnabled() { return S().entryLog; }
void SetEntryLogEnabled(bool on) { S().entryLog = on; }

void LogWrite(LogLevel, const char* tag, const char* file, int line, const char* fmt, ...)
{
    char msg[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    const char* base = strrchr(file, '/');
    base = base ? base + 1 : file;
    auto now = std::chrono::system_clock::now().time_since_epoch();
    long long us = std::chrono::duration_cast<std::chrono::microseconds>(now).count();
    LogState& s = S();
    std::lock_guard<std::mutex> lk(s.mu);
    fprintf(s.out, "[HCCL][%s][%lld.%06lld][pid %d][%s:%d] %s\n", tag, us / 1000000, us % 1000000, (int)getpid(),
            base, line, msg);
    fflush(s.out);
}

void ReportInputError(const char* code, const char* op, const char* param, const std::string& value,
                      const char* expect)
{
    LogWrite(LogLevel::ERROR, "ERROR", "input", 0, "[%s] op=%s parameter=%s value=%s expected=%s", code, op, param,
             value.c_str(), expect);
}

void DiagnoseRecord(const std::string& line)
{
    LogState& s = S();
    std::lock_guard<std::mutex> lk(s.mu);
    if (s.diag.size() >= s.diagCap) s.diag.pop_front();
    s.diag.push_back(line);
}

std::string DiagnoseDump()
{
    LogState& s = S();
    std::lock_guard<std::mutex> lk(s.mu);
    std::string out;
    for (auto& l : s.diag) {
        out += l;
        out += '\n';
    }
    return out;
}

const char* ResultString(HcclResult r)
{
    switch (r) {
        case HCCL_SUCCESS: return "HCCL_SUCCESS";
        case HCCL_E_PARA: return "HCCL_E_PARA (invalid parameter)";
        case HCCL_E_PTR: return "HCCL_E_PTR (null pointer)";
        case HCCL_E_MEMORY: return "HCCL_E_MEMORY";
        case HCCL_E_INTERNAL: return "HCCL_E_INTERNAL";
        case HCCL_E_NOT_SUPPORT: return "HCCL_E_NOT_SUPPORT";
        case HCCL_E_NOT_FOUND: return "HCCL_E_NOT_FOUND";
        case HCCL_E_UNAVAIL: return "HCCL_E_UNAVAIL (resource unavailable)";
        case HCCL_E_SYSCALL: return "HCCL_E_SYSCALL";
        case HCCL_E_TIMEOUT: return "HCCL_E_TIMEOUT";
        case HCCL_E_OPEN_FILE_FAILURE: return "HCCL_E_OPEN_FILE_FAILURE";
        case HCCL_E_TCP_CONNECT: return "HCCL_E_TCP_CONNECT";
        case HCCL_E_TCP_TRANSFER: return "HCCL_E_TCP_TRANSFER";
        case HCCL_E_RUNTIME: return "HCCL_E_RUNTIME (CUDA runtime error)";
        case HCCL_E_DRV: return "HCCL_E_DRV (CUDA driver error)";
        case HCCL_E_NETWORK: return "HCCL_E_NETWORK";
        case HCCL_E_AGAIN: return "HCCL_E_AGAIN";
        case HCCL_E_REMOTE: return "HCCL_E_REMOTE (a peer reported failure)";
        case HCCL_E_SUSPENDING: return "HCCL_E_SUSPENDING (communicator suspended)";
        case HCCL_E_OPRETRY_FAIL: return "HCCL_E_OPRETRY_FAIL";
        case HCCL_E_OOM: return "HCCL_E_OOM";
        default: return "HCCL_E_RESERVED";
    }
}

}  // namespace hccl
