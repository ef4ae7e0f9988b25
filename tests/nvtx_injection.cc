// A minimal NVTX injection library for the tests: NVTX v3 loads the library named by NVTX_INJECTION64_PATH on the
// first annotated call and hands it the callback tables; this one records every pushed range name and every pop as a
// line of the file named by HC_NVTX_LOG.
#include <cstdio>
#include <cstdlib>
#include <nvtx3/nvToolsExt.h>

static FILE *g_log = nullptr;

static int NVTX_API OnPushA(const char *message)
{
    if (g_log) { fprintf(g_log, "push %s\n", message); fflush(g_log); }
    return 0;
}
static int NVTX_API OnPop(void)
{
    if (g_log) { fprintf(g_log, "pop\n"); fflush(g_log); }
    return 0;
}

extern "C" int InitializeInjectionNvtx2(NvtxGetExportTableFunc_t getExportTable)
{
    const char *path = getenv("HC_NVTX_LOG");
    if (path) g_log = fopen(path, "w");
    const NvtxExportTableCallbacks *cb = (const NvtxExportTableCallbacks *)getExportTable(NVTX_ETID_CALLBACKS);
    if (!cb) return 0;
    NvtxFunctionTable table = nullptr;
    unsigned int size = 0;
    if (!cb->GetModuleFunctionTable(NVTX_CB_MODULE_CORE, &table, &size) || size <= NVTX_CBID_CORE_RangePop) return 0;
    *table[NVTX_CBID_CORE_RangePushA] = (NvtxFunctionPointer)OnPushA;
    *table[NVTX_CBID_CORE_RangePop] = (NvtxFunctionPointer)OnPop;
    return 1;
}
