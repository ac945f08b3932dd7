// Server side of the server <-> trainer hand-off: one POSIX shared segment holding the step
// counts and the CUDA IPC handles of every output buffer, plus two named semaphores per
// (device, pipe).  Byte-compatible with the trainer extension
// (training_backend/ipc_cuda_kernel.cu:30-95), which must keep working unchanged.
//
// Restates sampling_server/src/engine/ipc_service.cu and the POSIX half of
// engine/helper_multiprocess.cu:32-69.
#include "common.cuh"

#include <errno.h>
#include <fcntl.h>
#include <semaphore.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

namespace legion {

struct ShmLayout {  // shmStruct, engine/ipc_service.cu:28-31
    int32_t steps[3];
    cudaIpcMemHandle_t memHandle[LEGION_MAX_DEVICE][LEGION_INTERBATCH_CON][LEGION_MEMORY_USAGE];
};

}  // namespace legion

struct LegionIpcEnv {
    int32_t device_count;
    std::string shm_name;
    std::string sem_prefix;
    int shm_fd;
    volatile legion::ShmLayout *shm;
    // companion segment "<name>_ctr": the counter words of every finished batch in host memory, so that a
    // consumer need not read them from the device (the reference's trainer does two blocking device-to-host
    // copies per batch, training_backend/ipc_cuda_kernel.cu:194-203); consumers that do not know it ignore it
    int ctr_fd;
    volatile int32_t *ctr;  // [device][pipe][32]: node_counter[16], edge_counter[16]
    sem_t *semr[LEGION_MAX_DEVICE][LEGION_INTERBATCH_CON];
    sem_t *semw[LEGION_MAX_DEVICE][LEGION_INTERBATCH_CON];
    int32_t pipes[LEGION_MAX_DEVICE];
    int32_t raw_batch_size, epoch;
    int32_t train_step, valid_step, test_step;
    std::vector<int32_t> train_bs, valid_bs, test_bs;
};

using namespace legion;

static const char kDefaultShm[] = "simpleIPCshm";  // engine/ipc_service.cu:37
static constexpr size_t kCtrBytes = sizeof(int32_t) * LEGION_MAX_DEVICE * LEGION_INTERBATCH_CON * 32;

extern "C" int legion_ipc_layout(int64_t *segment_bytes, int64_t *handle_bytes, int64_t *handles_offset)
{
    if (segment_bytes) *segment_bytes = (int64_t)sizeof(ShmLayout);
    if (handle_bytes) *handle_bytes = (int64_t)sizeof(cudaIpcMemHandle_t);
    if (handles_offset) *handles_offset = (int64_t)offsetof(ShmLayout, memHandle);
    return LEGION_OK;
}

extern "C" int legion_ipc_create(LegionIpcEnv **out, int32_t device_count, const char *shm_name)
{
    LG_ARG(out != nullptr, "out is NULL");
    LG_ARG(device_count >= 1 && device_count <= LEGION_MAX_DEVICE, "device_count must be 1..8");
    LegionIpcEnv *e = new LegionIpcEnv();
    e->device_count = device_count;
    bool is_default = (shm_name == nullptr || shm_name[0] == 0 || strcmp(shm_name, kDefaultShm) == 0);
    e->shm_name = is_default ? kDefaultShm : shm_name;
    // the trainer derives the semaphore names from nothing but device and pipe
    // (ipc_cuda_kernel.cu:70-75); a non-default segment name gets its own family for tests
    e->sem_prefix = is_default ? "" : (e->shm_name + "_");
    e->shm = nullptr;
    e->raw_batch_size = e->epoch = 0;
    e->train_step = e->valid_step = e->test_step = 0;
    for (int d = 0; d < LEGION_MAX_DEVICE; ++d) {
        e->pipes[d] = 0;
        for (int p = 0; p < LEGION_INTERBATCH_CON; ++p) e->semr[d][p] = e->semw[d][p] = nullptr;
    }
    e->shm_fd = shm_open(e->shm_name.c_str(), O_RDWR | O_CREAT, 0777);
    if (e->shm_fd < 0) {
        set_error("legion_ipc_create: shm_open(%s): %s", e->shm_name.c_str(), strerror(errno));
        delete e;
        return LEGION_E_SYS;
    }
    if (ftruncate(e->shm_fd, sizeof(ShmLayout)) != 0) {
        set_error("legion_ipc_create: ftruncate: %s", strerror(errno));
        close(e->shm_fd);
        delete e;
        return LEGION_E_SYS;
    }
    void *addr = mmap(nullptr, sizeof(ShmLayout), PROT_READ | PROT_WRITE, MAP_SHARED, e->shm_fd, 0);
    if (addr == MAP_FAILED) {
        set_error("legion_ipc_create: mmap: %s", strerror(errno));
        close(e->shm_fd);
        delete e;
        return LEGION_E_SYS;
    }
    e->shm = (volatile ShmLayout *)addr;
    memset((void *)e->shm, 0, sizeof(ShmLayout));  // engine/ipc_service.cu:45
    // the companion segment is an extra: a failure here only means that consumers read the device counters
    e->ctr = nullptr;
    e->ctr_fd = shm_open((e->shm_name + "_ctr").c_str(), O_RDWR | O_CREAT, 0777);
    if (e->ctr_fd >= 0 && ftruncate(e->ctr_fd, kCtrBytes) == 0) {
        void *ca = mmap(nullptr, kCtrBytes, PROT_READ | PROT_WRITE, MAP_SHARED, e->ctr_fd, 0);
        if (ca != MAP_FAILED) {
            e->ctr = (volatile int32_t *)ca;
            memset((void *)e->ctr, 0, kCtrBytes);
        }
    }
    *out = e;
    return LEGION_OK;
}

// Counter words of the batch that was just finished on (dev, pipe), for consumers that read them from
// host memory; call before posting the batch.
extern "C" int legion_ipc_publish_counters(LegionIpcEnv *e, int32_t dev_id, int32_t pipe, const int32_t *node_counter,
                                           const int32_t *edge_counter)
{
    LG_ARG(e != nullptr && node_counter != nullptr && edge_counter != nullptr, "NULL pointer");
    LG_ARG(dev_id >= 0 && dev_id < LEGION_MAX_DEVICE && pipe >= 0 && pipe < LEGION_INTERBATCH_CON, "bad device or pipe");
    if (e->ctr == nullptr) return LEGION_OK;
    volatile int32_t *dst = e->ctr + ((size_t)dev_id * LEGION_INTERBATCH_CON + pipe) * 32;
    for (int i = 0; i < 16; ++i) {
        dst[i] = node_counter[i];
        dst[16 + i] = edge_counter[i];
    }
    return LEGION_OK;
}

extern "C" int legion_ipc_coordinate(LegionIpcEnv *e, const int32_t *train_num, const int32_t *valid_num,
                                     const int32_t *test_num, int32_t partition_count, int32_t raw_batch_size,
                                     int32_t epochs)
{
    LG_ARG(e != nullptr && train_num && valid_num && test_num, "NULL pointer");
    LG_ARG(partition_count >= 1 && partition_count <= LEGION_MAX_DEVICE, "partition_count must be 1..8");
    LG_ARG(raw_batch_size > 0 && epochs >= 0, "bad batch size or epoch count");
    e->raw_batch_size = raw_batch_size;
    e->epoch = epochs;
    int32_t min_train = 1000000000, max_valid = 0, max_test = 0;
    for (int i = 0; i < partition_count; ++i) {
        if (train_num[i] < min_train) min_train = train_num[i];
        if (valid_num[i] > max_valid) max_valid = valid_num[i];
        if (test_num[i] > max_test) max_test = test_num[i];
    }
    e->train_step = (min_train - 1) / raw_batch_size;  // engine/ipc_service.cu:82
    e->valid_step = (max_valid - 1) / 512 + 1;          // :99
    e->test_step = (max_test - 1) / 512 + 1;            // :112
    e->train_bs.assign(partition_count, raw_batch_size);
    e->valid_bs.resize(partition_count);
    e->test_bs.resize(partition_count);
    for (int i = 0; i < partition_count; ++i) {
        e->valid_bs[i] = (valid_num[i] - 1) / e->valid_step + 1;
        e->test_bs[i] = (test_num[i] - 1) / e->test_step + 1;
    }
    e->shm->steps[0] = e->train_step;
    e->shm->steps[1] = e->valid_step;
    e->shm->steps[2] = e->test_step;
    return LEGION_OK;
}

extern "C" int legion_ipc_steps(LegionIpcEnv *e, int32_t steps[3])
{
    LG_ARG(e != nullptr && steps != nullptr, "NULL pointer");
    steps[0] = e->shm->steps[0];
    steps[1] = e->shm->steps[1];
    steps[2] = e->shm->steps[2];
    return LEGION_OK;
}

extern "C" int legion_ipc_max_step(LegionIpcEnv *e)
{
    if (e == nullptr) return LEGION_E_ARG;
    return (e->train_step + e->valid_step) * e->epoch + e->test_step;  // engine/ipc_service.cu:130-132
}

extern "C" int legion_ipc_current_mode(LegionIpcEnv *e, int32_t global_batch_id)
{
    if (e == nullptr) return LEGION_E_ARG;
    if (global_batch_id < (e->train_step + e->valid_step) * e->epoch) {  // engine/ipc_service.cu:240-253
        int32_t eb = global_batch_id % (e->train_step + e->valid_step);
        return eb < e->train_step ? LEGION_TRAINMODE : LEGION_VALIDMODE;
    }
    return LEGION_TESTMODE;
}

extern "C" int legion_ipc_local_batch_id(LegionIpcEnv *e, int32_t global_batch_id)
{
    if (e == nullptr) return LEGION_E_ARG;
    if (global_batch_id < (e->train_step + e->valid_step) * e->epoch) {  // engine/ipc_service.cu:213-228
        int32_t eb = global_batch_id % (e->train_step + e->valid_step);
        return eb < e->train_step ? eb : eb - e->train_step;
    }
    return (global_batch_id - (e->train_step + e->valid_step) * e->epoch) % e->test_step;
}

extern "C" int legion_ipc_current_batchsize(LegionIpcEnv *e, int32_t dev_id, int32_t mode)
{
    if (e == nullptr || dev_id < 0 || dev_id >= (int)e->train_bs.size()) return LEGION_E_ARG;
    if (mode == LEGION_TRAINMODE) return e->train_bs[dev_id];  // engine/ipc_service.cu:230-238
    if (mode == LEGION_VALIDMODE) return e->valid_bs[dev_id];
    return e->test_bs[dev_id];
}

extern "C" int legion_ipc_open_semaphores(LegionIpcEnv *e, int32_t dev_id, int32_t pipes)
{
    LG_ARG(e != nullptr, "env is NULL");
    LG_ARG(dev_id >= 0 && dev_id < LEGION_MAX_DEVICE, "dev_id out of range");
    LG_ARG(pipes >= 1 && pipes <= LEGION_INTERBATCH_CON, "pipes must be 1 or 2");
    for (int i = 0; i < pipes; ++i) {
        std::string r = e->sem_prefix + "sem_r_" + std::to_string(dev_id) + "_" + std::to_string(i);
        std::string w = e->sem_prefix + "sem_w_" + std::to_string(dev_id) + "_" + std::to_string(i);
        e->semr[dev_id][i] = sem_open(r.c_str(), O_CREAT | O_RDWR, 0666, 0);  // engine/ipc_service.cu:181-192
        e->semw[dev_id][i] = sem_open(w.c_str(), O_CREAT | O_RDWR, 0666, 0);
        if (e->semr[dev_id][i] == SEM_FAILED || e->semw[dev_id][i] == SEM_FAILED) {
            set_error("legion_ipc_open_semaphores: sem_open: %s", strerror(errno));
            if (e->semr[dev_id][i] == SEM_FAILED) e->semr[dev_id][i] = nullptr;
            if (e->semw[dev_id][i] == SEM_FAILED) e->semw[dev_id][i] = nullptr;
            return LEGION_E_SYS;
        }
    }
    e->pipes[dev_id] = pipes;
    return LEGION_OK;
}

extern "C" int legion_ipc_publish_pool(LegionIpcEnv *e, LegionPool *pool, int32_t dev_id)
{
    LG_ARG(e != nullptr && pool != nullptr, "NULL handle");
    LG_ARG(dev_id >= 0 && dev_id < LEGION_MAX_DEVICE, "dev_id out of range");
    LG_ARG(pool->slots <= LEGION_INTERBATCH_CON, "the hand-off segment has two slots per device: create the pool with at most 2 slots");
    LG_CUDA(cudaSetDevice(pool->dev_id));
    for (int i = 0; i < pool->slots; ++i) {
        void *bufs[LEGION_MEMORY_USAGE] = { pool->pub_ids[i], pool->features[i], pool->pub_labels[i], pool->pub_agg_src[i],
                                            pool->pub_agg_dst[i], pool->pub_nc[i], pool->pub_ec[i] };
        for (int k = 0; k < LEGION_MEMORY_USAGE; ++k) {
            cudaIpcMemHandle_t h;
            LG_CUDA(cudaIpcGetMemHandle(&h, bufs[k]));  // engine/ipc_service.cu:163-169,203
            memcpy((void *)&e->shm->memHandle[dev_id][i][k], &h, sizeof(h));
        }
    }
    return legion_ipc_open_semaphores(e, dev_id, pool->slots);
}

extern "C" int legion_ipc_wait(LegionIpcEnv *e, int32_t dev_id, int32_t pipe, int32_t timeout_ms)
{
    LG_ARG(e != nullptr && dev_id >= 0 && dev_id < LEGION_MAX_DEVICE && pipe >= 0 && pipe < LEGION_INTERBATCH_CON,
           "bad device or pipe");
    sem_t *s = e->semr[dev_id][pipe];
    LG_ARG(s != nullptr, "semaphores of this device are not open");
    if (timeout_ms < 0) {
        while (sem_wait(s) != 0) {  // engine/ipc_service.cu:288-291
            if (errno != EINTR) { set_error("sem_wait: %s", strerror(errno)); return LEGION_E_SYS; }
        }
        return LEGION_OK;
    }
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    ts.tv_sec += timeout_ms / 1000;
    ts.tv_nsec += (long)(timeout_ms % 1000) * 1000000L;
    if (ts.tv_nsec >= 1000000000L) { ts.tv_sec += 1; ts.tv_nsec -= 1000000000L; }
    while (sem_timedwait(s, &ts) != 0) {
        if (errno == EINTR) continue;
        if (errno == ETIMEDOUT) {
            set_error("legion_ipc_wait: trainer of device %d did not release pipe %d within %d ms", dev_id, pipe,
                      timeout_ms);
            return LEGION_E_TIMEOUT;
        }
        set_error("sem_timedwait: %s", strerror(errno));
        return LEGION_E_SYS;
    }
    return LEGION_OK;
}

extern "C" int legion_ipc_post(LegionIpcEnv *e, int32_t dev_id, int32_t pipe)
{
    LG_ARG(e != nullptr && dev_id >= 0 && dev_id < LEGION_MAX_DEVICE && pipe >= 0 && pipe < LEGION_INTERBATCH_CON,
           "bad device or pipe");
    sem_t *s = e->semw[dev_id][pipe];
    LG_ARG(s != nullptr, "semaphores of this device are not open");
    if (sem_post(s) != 0) {  // engine/ipc_service.cu:283-286
        set_error("sem_post: %s", strerror(errno));
        return LEGION_E_SYS;
    }
    return LEGION_OK;
}

extern "C" int legion_ipc_destroy(LegionIpcEnv *e)
{
    if (e == nullptr) return LEGION_OK;
    for (int d = 0; d < LEGION_MAX_DEVICE; ++d) {
        for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) {
            if (e->semr[d][i]) sem_close(e->semr[d][i]);
            if (e->semw[d][i]) sem_close(e->semw[d][i]);
            if (e->semr[d][i] || e->semw[d][i]) {  // engine/ipc_service.cu:308-313
                std::string r = e->sem_prefix + "sem_r_" + std::to_string(d) + "_" + std::to_string(i);
                std::string w = e->sem_prefix + "sem_w_" + std::to_string(d) + "_" + std::to_string(i);
                sem_unlink(r.c_str());
                sem_unlink(w.c_str());
            }
        }
    }
    if (e->shm) munmap((void *)e->shm, sizeof(ShmLayout));
    if (e->shm_fd >= 0) close(e->shm_fd);
    shm_unlink(e->shm_name.c_str());
    if (e->ctr) munmap((void *)e->ctr, kCtrBytes);
    if (e->ctr_fd >= 0) close(e->ctr_fd);
    shm_unlink((e->shm_name + "_ctr").c_str());
    delete e;
    return LEGION_OK;
}

// Trainer side of one buffer: maps a handle read from the shared segment into this process
// (cudaIpcOpenMemHandle with cudaIpcMemLazyEnablePeerAccess, training_backend/ipc_cuda_kernel.cu:62-68).
extern "C" int legion_ipc_open_handle(const void *handle_bytes, void **dev_ptr)
{
    LG_ARG(handle_bytes != nullptr && dev_ptr != nullptr, "NULL pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_bytes, sizeof(h));
    LG_CUDA(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return LEGION_OK;
}

extern "C" int legion_ipc_close_handle(void *dev_ptr)
{
    LG_CUDA(cudaIpcCloseMemHandle(dev_ptr));  // training_backend/ipc_cuda_kernel.cu:143-149
    return LEGION_OK;
}

// Server side of one buffer: the 64-byte handle of a cudaMalloc allocation (engine/ipc_service.cu:163-169).
extern "C" int legion_ipc_get_handle(const void *dev_ptr, void *handle_bytes_out)
{
    LG_ARG(dev_ptr != nullptr && handle_bytes_out != nullptr, "NULL pointer");
    cudaIpcMemHandle_t h;
    LG_CUDA(cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr)));
    memcpy(handle_bytes_out, &h, sizeof(h));
    return LEGION_OK;
}

// ---- trainer side -----------------------------------------------------------------------------------------
// What the trainers' torch extension does (training_backend/ipc_cuda_kernel.cu:37-106,177-243 and
// ipc_service.cpp:44-92: initialize / get_next / get_block_size / get_steps / synchronize / finalize),
// without torch: the batch comes back as device pointers and counts.  Unlike the extension it does
// not copy the feature rows into a fresh tensor (ipc_cuda_kernel.cu:205-211): the rows stay where the
// server wrote them until legion_client_synchronize releases the pipe.
struct LegionClient {
    int32_t dev_id;
    std::string shm_name, sem_prefix;
    int shm_fd;
    volatile legion::ShmLayout *shm;
    void *buf[LEGION_INTERBATCH_CON][LEGION_MEMORY_USAGE];
    sem_t *semr[LEGION_INTERBATCH_CON], *semw[LEGION_INTERBATCH_CON];
    int current_pipe;
    int32_t *h_counters;  // pinned, 32 ints
    int ctr_fd;
    volatile int32_t *ctr;  // the server's companion segment, when there is one
};

extern "C" int legion_client_close(LegionClient *c)
{
    if (c == nullptr) return LEGION_OK;
    for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) {
        for (int k = 0; k < LEGION_MEMORY_USAGE; ++k)
            if (c->buf[i][k]) cudaIpcCloseMemHandle(c->buf[i][k]);  // ipc_cuda_kernel.cu:141-150
        if (c->semr[i]) sem_close(c->semr[i]);
        if (c->semw[i]) sem_close(c->semw[i]);
    }
    if (c->h_counters) cudaFreeHost(c->h_counters);
    if (c->ctr) munmap((void *)c->ctr, kCtrBytes);
    if (c->ctr_fd >= 0) close(c->ctr_fd);
    if (c->shm) munmap((void *)c->shm, sizeof(ShmLayout));
    if (c->shm_fd >= 0) close(c->shm_fd);
    delete c;
    return LEGION_OK;
}

// GPUIPCEnv::Initialize (ipc_cuda_kernel.cu:37-95) for the current device's slot `dev_id`.
extern "C" int legion_client_open(LegionClient **out, int32_t dev_id, const char *shm_name)
{
    LG_ARG(out != nullptr && dev_id >= 0 && dev_id < LEGION_MAX_DEVICE, "bad argument");
    LG_CUDA(cudaSetDevice(dev_id));
    LegionClient *c = new LegionClient();
    c->dev_id = dev_id;
    bool is_default = (shm_name == nullptr || shm_name[0] == 0 || strcmp(shm_name, kDefaultShm) == 0);
    c->shm_name = is_default ? kDefaultShm : shm_name;
    c->sem_prefix = is_default ? "" : (c->shm_name + "_");
    c->shm = nullptr;
    c->current_pipe = 0;
    c->h_counters = nullptr;
    c->ctr = nullptr;
    c->ctr_fd = -1;
    memset(c->buf, 0, sizeof(c->buf));
    for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) c->semr[i] = c->semw[i] = nullptr;
    c->shm_fd = shm_open(c->shm_name.c_str(), O_RDWR | O_CREAT, 0777);  // sharedMemoryCreate, as the trainer calls it
    if (c->shm_fd < 0 || ftruncate(c->shm_fd, sizeof(ShmLayout)) != 0) {
        set_error("legion_client_open: shared segment %s: %s", c->shm_name.c_str(), strerror(errno));
        legion_client_close(c);
        return LEGION_E_SYS;
    }
    void *addr = mmap(nullptr, sizeof(ShmLayout), PROT_READ | PROT_WRITE, MAP_SHARED, c->shm_fd, 0);
    if (addr == MAP_FAILED) {
        set_error("legion_client_open: mmap: %s", strerror(errno));
        legion_client_close(c);
        return LEGION_E_SYS;
    }
    c->shm = (volatile ShmLayout *)addr;
    // a server of this library also publishes the counters in host memory; the reference's does not
    c->ctr_fd = shm_open((c->shm_name + "_ctr").c_str(), O_RDONLY, 0);
    if (c->ctr_fd >= 0) {
        struct stat st;
        if (fstat(c->ctr_fd, &st) == 0 && (size_t)st.st_size >= kCtrBytes) {
            void *ca = mmap(nullptr, kCtrBytes, PROT_READ, MAP_SHARED, c->ctr_fd, 0);
            if (ca != MAP_FAILED) c->ctr = (volatile int32_t *)ca;
        }
    }
    for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) {
        for (int k = 0; k < LEGION_MEMORY_USAGE; ++k) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const void *)&c->shm->memHandle[dev_id][i][k], sizeof(h));
            cudaError_t e = cudaIpcOpenMemHandle(&c->buf[i][k], h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                set_error("legion_client_open: handle %d of pipe %d: %s (is the server ready?)", k, i, cudaGetErrorString(e));
                c->buf[i][k] = nullptr;
                legion_client_close(c);
                return LEGION_E_CUDA;
            }
        }
    }
    if (cudaMallocHost(reinterpret_cast<void **>(&c->h_counters), 128) != cudaSuccess) {
        set_error("legion_client_open: pinned allocation failed");
        legion_client_close(c);
        return LEGION_E_NOMEM;
    }
    for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) {
        std::string r = c->sem_prefix + "sem_r_" + std::to_string(dev_id) + "_" + std::to_string(i);
        std::string w = c->sem_prefix + "sem_w_" + std::to_string(dev_id) + "_" + std::to_string(i);
        c->semr[i] = sem_open(r.c_str(), O_CREAT | O_RDWR, 0666, 0);
        c->semw[i] = sem_open(w.c_str(), O_CREAT | O_RDWR, 0666, 0);
        if (c->semr[i] == SEM_FAILED || c->semw[i] == SEM_FAILED) {
            if (c->semr[i] == SEM_FAILED) c->semr[i] = nullptr;
            if (c->semw[i] == SEM_FAILED) c->semw[i] = nullptr;
            set_error("legion_client_open: sem_open: %s", strerror(errno));
            legion_client_close(c);
            return LEGION_E_SYS;
        }
        sem_post(c->semr[i]);  // both slots start free, ipc_cuda_kernel.cu:90
    }
    *out = c;
    return LEGION_OK;
}

extern "C" int legion_client_steps(LegionClient *c, int32_t steps[3])
{
    LG_ARG(c != nullptr && steps != nullptr, "NULL pointer");
    for (int i = 0; i < 3; ++i) steps[i] = c->shm->steps[i];  // get_steps, ipc_service.cpp:81-87
    return LEGION_OK;
}

// get_next + get_block_size (ipc_service.cpp:44-79, ipc_cuda_kernel.cu:177-243)
extern "C" int legion_client_get_next(LegionClient *c, int32_t timeout_ms, LegionBatchView *out)
{
    LG_ARG(c != nullptr && out != nullptr, "NULL pointer");
    sem_t *s = c->semw[c->current_pipe];
    if (timeout_ms < 0) {
        while (sem_wait(s) != 0)
            if (errno != EINTR) { set_error("sem_wait: %s", strerror(errno)); return LEGION_E_SYS; }
    } else {
        struct timespec ts;
        clock_gettime(CLOCK_REALTIME, &ts);
        ts.tv_sec += timeout_ms / 1000;
        ts.tv_nsec += (long)(timeout_ms % 1000) * 1000000L;
        if (ts.tv_nsec >= 1000000000L) { ts.tv_sec += 1; ts.tv_nsec -= 1000000000L; }
        while (sem_timedwait(s, &ts) != 0) {
            if (errno == EINTR) continue;
            if (errno == ETIMEDOUT) {
                set_error("legion_client_get_next: no batch within %d ms", timeout_ms);
                return LEGION_E_TIMEOUT;
            }
            set_error("sem_timedwait: %s", strerror(errno));
            return LEGION_E_SYS;
        }
    }
    LG_CUDA(cudaSetDevice(c->dev_id));
    void **b = c->buf[c->current_pipe];
    memset(out, 0, sizeof(*out));
    if (c->ctr != nullptr) {
        // written by the server before it posted this batch; the semaphore orders the two sides
        const volatile int32_t *src = c->ctr + ((size_t)c->dev_id * LEGION_INTERBATCH_CON + c->current_pipe) * 32;
        for (int i = 0; i < 16; ++i) {
            out->node_counter[i] = src[i];
            out->edge_counter[i] = src[16 + i];
        }
    } else {
        LG_CUDA(cudaMemcpyAsync(c->h_counters, b[5], 64, cudaMemcpyDeviceToHost, 0));
        LG_CUDA(cudaMemcpyAsync(c->h_counters + 16, b[6], 64, cudaMemcpyDeviceToHost, 0));
        LG_CUDA(cudaStreamSynchronize(0));
        memcpy(out->node_counter, c->h_counters, 64);
        memcpy(out->edge_counter, c->h_counters + 16, 64);
    }
    const int32_t *nc = out->node_counter, *ec = out->edge_counter;
    const int hops = nc[LEGION_INTRABATCH_CON * 3 - 1];
    if (hops < 0 || hops > LEGION_MAX_HOPS) {
        set_error("legion_client_get_next: counter block holds %d hops", hops);
        return LEGION_E_STATE;
    }
    out->hop_num = hops;
    out->n_ids = nc[LEGION_INTRABATCH_CON * 3 + hops];
    out->n_labels = nc[LEGION_INTRABATCH_CON * 3];
    out->ids = (const int32_t *)b[0];
    out->features = b[1];
    out->labels = (const int32_t *)b[2];
    for (int i = hops, j = 0; i > 0; --i, ++j) {  // last hop first, like the trainer unpacks it
        out->agg_src[j] = (const int32_t *)b[3] + ec[LEGION_INTRABATCH_CON * 4 + i];
        out->agg_dst[j] = (const int32_t *)b[4] + ec[LEGION_INTRABATCH_CON * 4 + i];
        out->n_edges[j] = ec[LEGION_INTRABATCH_CON * 3 + i];
        out->block_src[j] = nc[LEGION_INTRABATCH_CON * 3 + i];
        out->block_dst[j] = nc[LEGION_INTRABATCH_CON * 3 + i - 1];
    }
    return LEGION_OK;
}

// 1 when get_next takes the counters from the server's host segment, 0 when it reads the device buffers
extern "C" int legion_client_counters_on_host(LegionClient *c) { return (c != nullptr && c->ctr != nullptr) ? 1 : 0; }

// synchronize (ipc_service.cpp:89-91, ipc_cuda_kernel.cu:102-106): release the slot, move to the next
extern "C" int legion_client_synchronize(LegionClient *c)
{
    LG_ARG(c != nullptr, "client is NULL");
    if (sem_post(c->semr[c->current_pipe]) != 0) {
        set_error("sem_post: %s", strerror(errno));
        return LEGION_E_SYS;
    }
    c->current_pipe = (c->current_pipe + 1) % LEGION_INTERBATCH_CON;
    return LEGION_OK;
}
