/* hcomm_team_defs.h - handles and sizing request for SHMEM-style teams (reference: include/hcomm_team_defs.h). */
#ifndef HCOMM_TEAM_DEFS_H
#define HCOMM_TEAM_DEFS_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef uint64_t *HcommTeamHandle;
typedef uint64_t *HcommWindowHandle;
/* Number of 64-bit sync words of each kind that every member reserves for every other member. */
typedef struct {
    uint32_t signalCount;
    uint32_t counterCount;
    uint32_t barrierCount;
    uint32_t reserved[5];
} HcommTeamSyncMemRequirement;
#ifdef __cplusplus
}
#endif
#endif
