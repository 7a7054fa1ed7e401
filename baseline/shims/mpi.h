// SPDX-License-Identifier: Apache-2.0
/* Single-node stand-in for the handful of MPI calls the reference project makes (rank/size, a
 * broadcast from rank 0, the node-local split). MPI is not installed in this image; the ranks are
 * started with RANK / WORLD_SIZE / MASTER_PORT in the environment (torchrun or examples/launch.py)
 * and exchange broadcast payloads through files under /tmp keyed by MASTER_PORT. Only what
 * src/communication/communication.cpp and a driver's MPI_Init/MPI_Finalize need. */
#ifndef CS_BASELINE_MPI_SHIM_H
#define CS_BASELINE_MPI_SHIM_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Info;
#define MPI_COMM_WORLD 0
#define MPI_COMM_NULL (-1)
#define MPI_SUCCESS 0
#define MPI_MAX_PROCESSOR_NAME 256
#define MPI_CHAR 1
#define MPI_UINT16_T 2
#define MPI_DOUBLE 8
#define MPI_COMM_TYPE_SHARED 1
#define MPI_INFO_NULL 0
int MPI_Init(int *argc, char ***argv);
int MPI_Finalize(void);
int MPI_Comm_rank(MPI_Comm comm, int *rank);
int MPI_Comm_size(MPI_Comm comm, int *size);
int MPI_Get_processor_name(char *name, int *len);
int MPI_Bcast(void *buffer, int count, MPI_Datatype type, int root, MPI_Comm comm);
int MPI_Comm_split_type(MPI_Comm comm, int split_type, int key, MPI_Info info, MPI_Comm *out);
int MPI_Comm_free(MPI_Comm *comm);
int MPI_Barrier(MPI_Comm comm);
/* max over ranks of one double (all ranks receive it) */
int MPI_Shim_max_double(double *value);
#ifdef __cplusplus
}
#endif
#endif
