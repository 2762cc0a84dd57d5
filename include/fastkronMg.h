/*
 * fastkronMg.h -- multi-GPU GeMKM entry points, same ABI as
 * abhijangda/fastkron's include/fastkronMg.h:8-18.
 *
 * One process drives `gpus` devices of one node.  X, the result and the
 * temporaries are per-device buffers; device g = r*gpusInK + c owns rows
 * [r*M/gpusInM, (r+1)*M/gpusInM) and columns [c*K/gpusInK, (c+1)*K/gpusInK) of
 * the global matrix, every factor is replicated on every device.  fp32,
 * row-major, opX = opF = N only, like the reference.
 */
#pragma once

#include <stdint.h>
#include <stddef.h>

#include "fastkron.h"

#ifdef __cplusplus
#define FASTKRON_MG_DEFAULT(v) = v
extern "C" {
#else
#define FASTKRON_MG_DEFAULT(v)
#endif

/* `streams` points to an array of `gpus` cudaStream_t, stream g on device g.
 * gpusInM * gpusInK must equal gpus (otherwise fastKronInvalidArgument); the
 * defaults are the reference's: gpusInM = -1 selects 1, gpusInK = -1 selects 2.
 * gpuLocalKrons (factors applied between two exchanges in the reference) is
 * accepted and ignored: the schedule here always uses two exchanges.
 * (reference: include/fastkronMg.h:10, src/kernel_db/cuda_kernel_db.cu:62-186) */
fastKronError fastKronMgInitCUDA(fastKronHandle handle, void* streams, int gpus,
                                 int gpusInM FASTKRON_MG_DEFAULT(-1),
                                 int gpusInK FASTKRON_MG_DEFAULT(-1),
                                 int gpuLocalKrons FASTKRON_MG_DEFAULT(-1));

/* x[g], result[g], temp1[g], temp2[g] are device-g buffers sized by gekmmSizes()
 * called after fastKronMgInitCUDA; kronMats[g*NumKronMats + i] is factor i on
 * device g.  Blocking: returns after every device finished.  The result is left
 * distributed in result[g] with the same block layout as X.
 * (reference: include/fastkronMg.h:13-15, src/handle/distrib_handle.cu:504-521) */
fastKronError fastKronMgSGEMM(fastKronHandle handle, const uint32_t NumKronMats,
                              void* x[], void* kronMats[], void* result[],
                              uint32_t M, uint32_t N, uint32_t K,
                              uint32_t KronMatCols[], uint32_t KronMatRows[],
                              void* temp1[], void* temp2[], void* stream);

/* Allocate dX[g] on each device and scatter the host matrix hX (M x K, row-major)
 * into the block layout above; the caller frees dX[g] with cudaFree.
 * (reference: include/fastkronMg.h:16, src/handle/distrib_handle.cu:428-464) */
fastKronError fastKronMgAllocX(fastKronHandle handle, void* dX[], void* hX,
                               uint32_t M, uint32_t K);

/* Gather the distributed result blocks dY[g] into the host matrix hY
 * (M x prod KronMatCols, row-major).
 * (reference: include/fastkronMg.h:17, src/handle/distrib_handle.cu:466-502) */
fastKronError fastKronMgGatherY(fastKronHandle handle, void* dY[], void* hY,
                                uint32_t M, uint32_t K, uint32_t NumKronMats,
                                uint32_t KronMatCols[], uint32_t KronMatRows[]);

#ifdef __cplusplus
}
#endif
