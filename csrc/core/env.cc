#include "env.h"

#include <cstdlib>
#include <mutex>

#include "log.h"

namespace hc {

template <typename T>
void EnvField<T>::Load(const std::function<bool(const std::string &, T &)> &parser,
                       const std::function<bool(const T &)> &validator)
{
    const char *raw = getenv(name);
    fromEnv = false;
    if (raw == nullptr || *raw == '\0') return;
    T parsed{};
    if (!parser(raw, parsed)) {
        HCCL_WARNING("env %s=\"%s\" is malformed, default kept", name, raw);
        return;
    }
    if (validator && !validator(parsed)) {
        HCCL_WARNING("env %s=\"%s\" is out of range, default kept", name, raw);
        return;
    }
    value = parsed;
    fromEnv = true;
}

namespace {
bool ParseInt(const std::string &s, int32_t &out)
{
    char *end = nullptr;
    long v = strtol(s.c_str(), &end, 10);
    if (end == s.c_str() || *end != '\0') return false;
    out = (int32_t)v;
    return true;
}
bool ParseU32(const std::string &s, uint32_t &out)
{
    int32_t v;
    if (!ParseInt(s, v) || v < 0) return false;
    out = (uint32_t)v;
    return true;
}
bool ParseStr(const std::string &s, std::string &out)
{
    out = s;
    return true;
}
// Accepts 0/1/2 and the words false/true/strict (HCCL_DETERMINISTIC).
bool ParseDeterministic(const std::string &s, int32_t &out)
{
    if (s == "false" || s == "FALSE") { out = 0; return true; }
    if (s == "true" || s == "TRUE") { out = 1; return true; }
    if (s == "strict" || s == "STRICT") { out = 2; return true; }
    return ParseInt(s, out);
}
// "AI_CPU", "AIV", "HOST", "HOST_TS", "CCU_MS", "CCU_SCHED", "AIV_ONLY" or a number.
bool ParseExpansion(const std::string &s, int32_t &out)
{
    static const struct { const char *k; int v; } tbl[] = {{"AI_CPU", 2}, {"AIV", 3}, {"HOST", 1}, {"HOST_TS", 2},
                                                          {"CCU_MS", 5}, {"CCU_SCHED", 6}, {"AIV_ONLY", 4}};
    for (auto &e : tbl)
        if (s == e.k) { out = e.v; return true; }
    return ParseInt(s, out);
}
std::mutex g_mu;
EnvConfig *g_cfg = nullptr;
}  // namespace

bool ParsePortRange(const std::string &s, int &lo, int &hi)
{
    auto dash = s.find('-');
    int32_t a, b;
    if (dash == std::string::npos) {
        if (!ParseInt(s, a)) return false;
        lo = hi = a;
    } else {
        if (!ParseInt(s.substr(0, dash), a) || !ParseInt(s.substr(dash + 1), b)) return false;
        lo = a;
        hi = b;
    }
    return lo > 0 && hi >= lo && hi < 65536;
}

void EnvConfig::LoadAll()
{
    buffSizeMB.Load(ParseU32, [](const uint32_t &v) { return v >= 1 && v <= 65536; });
    algo.Load(ParseStr);
    opExpansionMode.Load(ParseExpansion, [](const int32_t &v) { return v >= 0 && v <= 6; });
    deterministic.Load(ParseDeterministic, [](const int32_t &v) { return v >= 0 && v <= 2; });
    execTimeoutSec.Load(ParseInt, [](const int32_t &v) { return v >= 0 && v <= 2147483; });
    connectTimeoutSec.Load(ParseInt, [](const int32_t &v) { return v >= 1 && v <= 7200; });
    ifIp.Load(ParseStr);
    ifBasePort.Load(ParseInt, [](const int32_t &v) { return v >= 1024 && v < 65520; });
    socketIfname.Load(ParseStr);
    socketFamily.Load(ParseStr, [](const std::string &v) { return v == "AF_INET" || v == "AF_INET6"; });
    hostPortRange.Load(ParseStr, [](const std::string &v) { int a, b; return v == "auto" || ParsePortRange(v, a, b); });
    whitelistDisable.Load(ParseInt);
    whitelistFile.Load(ParseStr);
    opRetryEnable.Load(ParseInt);
    opRetryParams.Load(ParseStr);
    entryLogEnable.Load(ParseInt);
    diagnoseEnable.Load(ParseInt);
    heartbeatMs.Load(ParseInt, [](const int32_t &v) { return v >= 0; });
    heartbeatLostMs.Load(ParseInt, [](const int32_t &v) { return v > 0; });
    simulate.Load(ParseInt);
    nvlsEnable.Load(ParseInt);
    maxCtas.Load(ParseInt, [](const int32_t &v) { return v >= 0 && v <= 1024; });
    forceCtas.Load(ParseInt, [](const int32_t &v) { return v >= 0 && v <= 1024; });
    llMaxBytes.Load(ParseInt, [](const int32_t &v) { return v >= 0 && v <= 1048576; });
    llMaxRecvBytes.Load(ParseInt, [](const int32_t &v) { return v >= 0; });
    tuneFile.Load(ParseStr);
    symStrideGB.Load(ParseInt, [](const int32_t &v) { return v >= 0 && v <= 4096; });
}

const EnvConfig &EnvConfig::Get()
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_cfg) {
        g_cfg = new EnvConfig();
        g_cfg->LoadAll();
    }
    return *g_cfg;
}

void EnvConfig::Reload()
{
    std::lock_guard<std::mutex> lk(g_mu);
    delete g_cfg;
    g_cfg = new EnvConfig();
    g_cfg->LoadAll();
    LogReload();
}

template struct EnvField<int32_t>;
template struct EnvField<uint32_t>;
template struct EnvField<std::string>;

}  // namespace hc
