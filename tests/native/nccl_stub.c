/* A stand-in for the NCCL shared library, loaded by path through qmm_llama_tp_unique_id /
 * qmm_llama_tp_init, for testing failure detection around the prefill collectives WITHOUT a second
 * GPU, a real communicator or any GPU fault.  Collectives move no data.  Behaviour is set by
 * environment variables read at each call:
 *   NCCL_STUB_BUSY_MS=<ms>      every all-reduce enqueues a HOST function on the caller's stream that
 *                               sleeps this long (the stream stays busy; the GPU is idle and healthy)
 *   NCCL_STUB_ASYNC_ERROR=<n>   ncclCommGetAsyncError reports n once an all-reduce has been enqueued
 *   NCCL_STUB_LOG=<path>        one line per call is appended to this file
 * Build: gcc -shared -fPIC -I<cuda>/include nccl_stub.c -o libnccl_stub.so -L<cuda>/lib64 -lcudart */
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef struct {
    char bytes[128];
} stub_unique_id;

static int g_reduces = 0;
static int g_comm_token = 0;

static void stub_log(const char* what)
{
    const char* path = getenv("NCCL_STUB_LOG");
    if (path && path[0]) {
        FILE* f = fopen(path, "a");
        if (f) {
            fprintf(f, "%s\n", what);
            fclose(f);
        }
    }
}

static void CUDART_CB stub_sleep(void* arg)
{
    const long ms = (long)(size_t)arg;
    struct timespec ts = {ms / 1000, (ms % 1000) * 1000000L};
    nanosleep(&ts, NULL);
}

int ncclGetUniqueId(stub_unique_id* id)
{
    memset(id->bytes, 0, sizeof id->bytes);
    strcpy(id->bytes, "nccl-stub-unique-id");
    stub_log("ncclGetUniqueId");
    return 0;
}

int ncclCommInitRank(void** comm, int nranks, stub_unique_id id, int rank)
{
    (void)nranks;
    (void)rank;
    if (strcmp(id.bytes, "nccl-stub-unique-id") != 0) {
        return 5; /* ncclInvalidArgument */
    }
    *comm = &g_comm_token;
    g_reduces = 0;
    stub_log("ncclCommInitRank");
    return 0;
}

int ncclAllReduce(const void* send, void* recv, size_t count, int dtype, int op, void* comm, void* stream)
{
    (void)send;
    (void)recv;
    (void)count;
    (void)dtype;
    (void)op;
    (void)comm;
    const char* busy = getenv("NCCL_STUB_BUSY_MS");
    if (busy && atol(busy) > 0) {
        if (cudaLaunchHostFunc((cudaStream_t)stream, stub_sleep, (void*)(size_t)atol(busy)) != cudaSuccess) {
            return 1; /* ncclUnhandledCudaError */
        }
    }
    ++g_reduces;
    stub_log("ncclAllReduce");
    return 0;
}

int ncclAllGather(const void* send, void* recv, size_t count, int dtype, void* comm, void* stream)
{
    (void)send;
    (void)recv;
    (void)count;
    (void)dtype;
    (void)comm;
    (void)stream;
    stub_log("ncclAllGather");
    return 0;
}

int ncclCommGetAsyncError(void* comm, int* async_error)
{
    (void)comm;
    const char* err = getenv("NCCL_STUB_ASYNC_ERROR");
    *async_error = (err && g_reduces > 0) ? atoi(err) : 0;
    return 0;
}

int ncclCommAbort(void* comm)
{
    (void)comm;
    stub_log("ncclCommAbort");
    return 0;
}

int ncclCommDestroy(void* comm)
{
    (void)comm;
    stub_log("ncclCommDestroy");
    return 0;
}
