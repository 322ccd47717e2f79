// In-process stand-in for the handful of MPI C calls the MPI adapter makes, so that the adapter
// is compiled and exercised where no MPI is installed. "Ranks" are threads of one process: each
// thread binds itself to a rank of the world before it calls anything else. This is NOT an MPI
// implementation; only what src/bootstrap/mpi/mpi_bootstrap.cc uses exists.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

typedef struct FakeMpiWorld* MPI_Comm;
typedef int MPI_Datatype;

#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_MAX_ERROR_STRING 256
#define MPI_BYTE 1
#define MPI_INT 2

int MPI_Initialized(int* flag);
int MPI_Finalized(int* flag);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Allgather(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                  MPI_Datatype recvtype, MPI_Comm comm);
int MPI_Barrier(MPI_Comm comm);
int MPI_Error_string(int errorcode, char* string, int* resultlen);

/* Test controls. */
MPI_Comm fake_mpi_create_world(int size);
void fake_mpi_destroy_world(MPI_Comm world);
void fake_mpi_bind_thread(MPI_Comm world, int rank);   /* the calling thread becomes `rank` */
void fake_mpi_set_initialized(int initialized, int finalized);
void fake_mpi_fail_next_allgather(MPI_Comm world, int code); /* every rank's next MPI_Allgather returns `code` */

#ifdef __cplusplus
}
#endif
