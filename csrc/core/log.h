// log.h - leveled, category-masked logging and structured error reports.
//
// Level comes from HCCL_LOG_LEVEL or ASCEND_LOG_LEVEL (0 debug, 1 info, 2 warning, 3 error; default 2).
// HCCL_DEBUG_CONFIG is a comma list of categories (ALG, TASK, RESOURCE, KERNEL, BOOT) whose debug lines
// are printed even when the level is above debug (reference: common/debug/config/config_log.cc:41-47).
// RPT_ERR attaches a catalogue code "EI00xx" the way RPT_INPUT_ERR does in the reference.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <string>

namespace hc {

enum LogLevel { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARN = 2, LOG_ERROR = 3, LOG_RUN = 4 };
enum LogCat : uint32_t { CAT_NONE = 0, CAT_ALG = 1, CAT_TASK = 2, CAT_RESOURCE = 4, CAT_KERNEL = 8, CAT_BOOT = 16 };

bool LogEnabled(LogLevel lvl, uint32_t cat);
void LogWrite(LogLevel lvl, const char *file, int line, const char *fmt, ...) __attribute__((format(printf, 4, 5)));
void LogReload();                 // re-read the environment (tests)
std::string LogLastError();      // newest ERROR line of this thread, for HcclDiagDump
void ReportError(const char *code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

}  // namespace hc

#define HC_LOG(lvl, cat, ...)                                             \
    do {                                                                  \
        if (::hc::LogEnabled(lvl, cat)) ::hc::LogWrite(lvl, __FILE__, __LINE__, __VA_ARGS__); \
    } while (0)
#define HCCL_DEBUG(...) HC_LOG(::hc::LOG_DEBUG, ::hc::CAT_NONE, __VA_ARGS__)
#define HCCL_DEBUG_CAT(cat, ...) HC_LOG(::hc::LOG_DEBUG, cat, __VA_ARGS__)
#define HCCL_INFO(...) HC_LOG(::hc::LOG_INFO, ::hc::CAT_NONE, __VA_ARGS__)
#define HCCL_WARNING(...) HC_LOG(::hc::LOG_WARN, ::hc::CAT_NONE, __VA_ARGS__)
#define HCCL_ERROR(...) HC_LOG(::hc::LOG_ERROR, ::hc::CAT_NONE, __VA_ARGS__)
#define HCCL_RUN_INFO(...) HC_LOG(::hc::LOG_RUN, ::hc::CAT_NONE, __VA_ARGS__)
#define RPT_ERR(code, ...) ::hc::ReportError(code, __VA_ARGS__)

// Early-return helpers.
#define CHK_PTR_NULL(p)                                        \
    do {                                                       \
        if ((p) == nullptr) {                                  \
            RPT_ERR("EI0003", "null pointer: %s", #p);         \
            return HCCL_E_PTR;                                 \
        }                                                      \
    } while (0)
#define CHK_RET(expr)                                          \
    do {                                                       \
        HcclResult _r = (expr);                                \
        if (_r != HCCL_SUCCESS) {                              \
            HCCL_ERROR("%s failed: %d", #expr, (int)_r);       \
            return _r;                                         \
        }                                                      \
    } while (0)
#define CHK_PRT_RET(cond, ret, ...)                            \
    do {                                                       \
        if (cond) {                                            \
            HCCL_ERROR(__VA_ARGS__);                           \
            return ret;                                        \
        }                                                      \
    } while (0)
