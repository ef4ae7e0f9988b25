#include "log.h"

#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>

namespace hc {
namespace {
std::atomic<int> g_level{-1};
std::atomic<uint32_t> g_cats{0};
thread_local std::string t_lastError;

void Load()
{
    int lvl = LOG_WARN;
    const char *s = getenv("HCCL_LOG_LEVEL");
    if (!s) s = getenv("ASCEND_LOG_LEVEL");
    if (s && *s >= '0' && *s <= '3') lvl = *s - '0';
    uint32_t cats = 0;
    if (const char *c = getenv("HCCL_DEBUG_CONFIG")) {
        std::string v(c);
        auto has = [&](const char *k) { return v.find(k) != std::string::npos; };
        if (has("ALG")) cats |= CAT_ALG;
        if (has("TASK")) cats |= CAT_TASK;
        if (has("RESOURCE")) cats |= CAT_RESOURCE;
        if (has("KERNEL") || has("AIV_OPS_EXC")) cats |= CAT_KERNEL;
        if (has("BOOT")) cats |= CAT_BOOT;
    }
    g_cats.store(cats);
    g_level.store(lvl);
}
}  // namespace

void LogReload() { Load(); }

bool LogEnabled(LogLevel lvl, uint32_t cat)
{
    if (g_level.load(std::memory_order_relaxed) < 0) Load();
    if (lvl == LOG_RUN) return g_level.load() <= LOG_INFO;
    if ((int)lvl >= g_level.load(std::memory_order_relaxed)) return true;
    return cat != 0 && (g_cats.load(std::memory_order_relaxed) & cat) != 0;
}

void LogWrite(LogLevel lvl, const char *file, int line, const char *fmt, ...)
{
    static const char *names[] = {"DEBUG", "INFO", "WARNING", "ERROR", "RUN"};
    char msg[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    const char *base = strrchr(file, '/');
    base = base ? base + 1 : file;
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    struct tm tmv;
    localtime_r(&ts.tv_sec, &tmv);
    char line_buf[1280];
    snprintf(line_buf, sizeof(line_buf), "[%s] HCCL(%d,%ld) %02d:%02d:%02d.%03ld [%s:%d] %s\n", names[lvl], (int)getpid(),
             (long)syscall(SYS_gettid), tmv.tm_hour, tmv.tm_min, tmv.tm_sec, ts.tv_nsec / 1000000, base, line, msg);
    if (lvl == LOG_ERROR) t_lastError = msg;
    fputs(line_buf, stderr);
}

std::string LogLastError() { return t_lastError; }

void ReportError(const char *code, const char *fmt, ...)
{
    char msg[900];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    LogWrite(LOG_ERROR, "report", 0, "[%s] %s", code, msg);
}

}  // namespace hc
