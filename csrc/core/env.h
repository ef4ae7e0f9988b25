// env.h - typed environment configuration parsed once per process.
//
// Each knob is an EnvField{name, default, parser, validator}; a value that fails to parse or
// validate falls back to the default with a warning, as the reference's EnvField<T> does
// (src/base_comm/config_mgr/base_config.h:103-160).  EnvConfig::Get() is the process snapshot;
// EnvConfig::Reload() re-reads it (tests only).
#pragma once
#include <cstdint>
#include <functional>
#include <string>

namespace hc {

template <typename T>
struct EnvField {
    const char *name;
    T value;
    bool fromEnv = false;
    EnvField(const char *n, T def) : name(n), value(def) {}
    // parser returns false on malformed text; validator false on out-of-range.
    void Load(const std::function<bool(const std::string &, T &)> &parser,
              const std::function<bool(const T &)> &validator = nullptr);
};

struct EnvConfig {
    EnvField<uint32_t> buffSizeMB{"HCCL_BUFFSIZE", 200};
    EnvField<std::string> algo{"HCCL_ALGO", ""};
    EnvField<int32_t> opExpansionMode{"HCCL_OP_EXPANSION_MODE", 0};
    EnvField<int32_t> deterministic{"HCCL_DETERMINISTIC", 0};
    EnvField<int32_t> execTimeoutSec{"HCCL_EXEC_TIMEOUT", 1836};
    EnvField<int32_t> connectTimeoutSec{"HCCL_CONNECT_TIMEOUT", 120};
    EnvField<std::string> ifIp{"HCCL_IF_IP", ""};
    EnvField<int32_t> ifBasePort{"HCCL_IF_BASE_PORT", 0};
    EnvField<std::string> socketIfname{"HCCL_SOCKET_IFNAME", ""};
    EnvField<std::string> socketFamily{"HCCL_SOCKET_FAMILY", "AF_INET"};
    EnvField<std::string> hostPortRange{"HCCL_HOST_SOCKET_PORT_RANGE", ""};
    EnvField<int32_t> whitelistDisable{"HCCL_WHITELIST_DISABLE", 1};
    EnvField<std::string> whitelistFile{"HCCL_WHITELIST_FILE", ""};
    EnvField<int32_t> opRetryEnable{"HCCL_OP_RETRY_ENABLE", 0};
    EnvField<std::string> opRetryParams{"HCCL_OP_RETRY_PARAMS", "MaxCnt:1,HoldTime:5000,IntervalTime:1000"};
    EnvField<int32_t> entryLogEnable{"HCCL_ENTRY_LOG_ENABLE", 0};
    EnvField<int32_t> diagnoseEnable{"HCCL_DIAGNOSE_ENABLE", 0};
    EnvField<int32_t> heartbeatMs{"HCCL_HEARTBEAT_INTERVAL_MS", 0};   // 0 = heartbeat thread off
    EnvField<int32_t> heartbeatLostMs{"HCCL_HEARTBEAT_LOST_MS", 30000};
    // B200-specific knobs
    EnvField<int32_t> simulate{"HCCL_SIM", -1};             // 1 force host simulator, 0 force CUDA, -1 auto
    EnvField<int32_t> nvlsEnable{"HCCL_NVLS_ENABLE", 1};
    EnvField<int32_t> maxCtas{"HCCL_MAX_CTAS", 0};          // upper bound of CTAs per collective kernel; 0 = selector decides
    EnvField<int32_t> forceCtas{"HCCL_FORCE_CTAS", 0};      // exact CTA count (tuning runs); 0 = off
    EnvField<int32_t> llMaxBytes{"HCCL_LL_MAX_BYTES", 1048576};            // largest block (bytes per peer) the flag-in-data kernel serves; 0 = never
    EnvField<int32_t> llMaxRecvBytes{"HCCL_LL_MAX_RECV_BYTES", 1048576};   // and the most one rank may receive that way, (ranks - 1) x block
    EnvField<std::string> tuneFile{"HCCL_TUNE_FILE", ""};   // measured bus-bandwidth table (JSON)
    EnvField<int32_t> symStrideGB{"HCCL_SYM_STRIDE_GB", 0};

    static const EnvConfig &Get();
    static void Reload();
    void LoadAll();
};

// "60000-60015" style ranges; returns false when malformed.
bool ParsePortRange(const std::string &s, int &lo, int &hi);

}  // namespace hc
