// SPDX-License-Identifier: Apache-2.0
/* See mpi.h in this directory. File-based collectives for ranks of one node. */
#include "mpi.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

static int env_int(const char *name, int fallback) {
  const char *v = getenv(name);
  return v ? atoi(v) : fallback;
}
static int g_seq = 0;
/* CS_MPISHIM_KEY (set by the launcher to something unique per run) keeps runs apart. */
static void path_of(char *out, size_t n, const char *kind, int seq, int rank) {
  const char *key = getenv("CS_MPISHIM_KEY");
  snprintf(out, n, "/tmp/cs_mpishim_%s_%d_%s_%d_%d", key ? key : "run", env_int("MASTER_PORT", 29500), kind, seq, rank);
}
static char g_written[64][512];
static int g_num_written = 0;
static int type_size(MPI_Datatype t) { return t == MPI_UINT16_T ? 2 : (t == MPI_DOUBLE ? 8 : 1); }

static void write_file(const char *path, const void *data, size_t n) {
  char tmp[512];
  snprintf(tmp, sizeof(tmp), "%s.tmp", path);
  FILE *f = fopen(tmp, "wb");
  if (!f) abort();
  fwrite(data, 1, n, f);
  fclose(f);
  rename(tmp, path); /* atomic publish */
  if (g_num_written < 64) strncpy(g_written[g_num_written++], path, 511);
}
static void read_file(const char *path, void *data, size_t n) {
  for (int tries = 0; tries < 600000; ++tries) { /* up to ~10 minutes */
    FILE *f = fopen(path, "rb");
    if (f) {
      const size_t got = fread(data, 1, n, f);
      fclose(f);
      if (got == n) return;
    }
    usleep(1000);
  }
  fprintf(stderr, "mpi shim: timed out waiting for %s\n", path);
  abort();
}

int MPI_Init(int *argc, char ***argv) { (void)argc; (void)argv; return MPI_SUCCESS; }
int MPI_Finalize(void) {
  /* everyone has read everything once the last barrier is through; each rank removes its own files */
  MPI_Barrier(MPI_COMM_WORLD);
  usleep(200000);
  for (int i = 0; i < g_num_written; ++i) unlink(g_written[i]);
  g_num_written = 0;
  return MPI_SUCCESS;
}
int MPI_Comm_rank(MPI_Comm comm, int *rank) { (void)comm; *rank = env_int("RANK", 0); return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm comm, int *size) { (void)comm; *size = env_int("WORLD_SIZE", 1); return MPI_SUCCESS; }
int MPI_Get_processor_name(char *name, int *len) {
  strcpy(name, "localhost");
  *len = 9;
  return MPI_SUCCESS;
}
int MPI_Bcast(void *buffer, int count, MPI_Datatype type, int root, MPI_Comm comm) {
  (void)comm;
  const int rank = env_int("RANK", 0), size = env_int("WORLD_SIZE", 1);
  if (size <= 1) return MPI_SUCCESS;
  char path[512];
  const int seq = g_seq++;
  path_of(path, sizeof(path), "bcast", seq, root);
  const size_t n = (size_t)count * type_size(type);
  if (rank == root) write_file(path, buffer, n); else read_file(path, buffer, n);
  return MPI_SUCCESS;
}
int MPI_Comm_split_type(MPI_Comm comm, int split_type, int key, MPI_Info info, MPI_Comm *out) {
  (void)comm; (void)split_type; (void)key; (void)info;
  *out = 1; /* all ranks share the node */
  return MPI_SUCCESS;
}
int MPI_Comm_free(MPI_Comm *comm) { *comm = MPI_COMM_NULL; return MPI_SUCCESS; }
int MPI_Shim_max_double(double *value) {
  const int rank = env_int("RANK", 0), size = env_int("WORLD_SIZE", 1);
  if (size <= 1) return MPI_SUCCESS;
  char path[512];
  const int seq = g_seq++;
  path_of(path, sizeof(path), "max", seq, rank);
  write_file(path, value, sizeof(double));
  double best = *value;
  for (int r = 0; r < size; ++r) {
    double v;
    path_of(path, sizeof(path), "max", seq, r);
    read_file(path, &v, sizeof(double));
    if (v > best) best = v;
  }
  *value = best;
  return MPI_SUCCESS;
}
int MPI_Barrier(MPI_Comm comm) {
  (void)comm;
  double zero = 0;
  return MPI_Shim_max_double(&zero);
}
