// Per-device state shared by the launchers: the error word written by kernels
// whose bounded waits ran out, cached device properties, staging buffers for
// the host-buffer entry point, and the library-wide shutdown.
#include "common.cuh"
#include "runtime.cuh"
#include <mutex>

namespace b200wmma
{
    namespace
    {
        constexpr int MAX_DEVICES = 64;

        struct DeviceState
        {
            uint32_t* status  = nullptr; // device uint32_t[4]
            int       smCount = 0;
            void*     scratch = nullptr; // general scratch (GEMV partial sums ...)
            size_t    scratchBytes = 0;
            void*     splitWs      = nullptr; // partial accumulators of split GEMM tiles
            size_t    splitWsBytes = 0;
            uint32_t* splitCtr     = nullptr; // 256 arrival counters
            void*     stage[4]      = {nullptr, nullptr, nullptr, nullptr}; // A, B, C, D staging
            size_t    stageBytes[4] = {0, 0, 0, 0};
            HostPipe  pipe;
            unsigned int* counters = nullptr; // 64 launch counters, 32 bytes apart
            cudaStream_t  counterStream[64] = {}; // stream that owns counter i
            unsigned int  counterStreams    = 0;
            std::mutex    hostCall; // serialises the host-buffer entry point per device
        };

        std::mutex  g_mutex;
        DeviceState g_dev[MAX_DEVICES];

        DeviceState* current()
        {
            int dev = -1;
            if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
            {
                (void)cudaGetLastError();
                return nullptr;
            }
            return &g_dev[dev];
        }
    } // namespace

    EncodeFn tensorMapEncoder()
    {
        static EncodeFn       fn = nullptr;
        static std::once_flag once;
        std::call_once(once, [] {
            void*                           sym = nullptr;
            cudaDriverEntryPointQueryResult q;
            if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q)
                   == cudaSuccess
               && q == cudaDriverEntryPointSuccess)
                fn = reinterpret_cast<EncodeFn>(sym);
            else
                (void)cudaGetLastError();
        });
        return fn;
    }

    uint32_t* deviceStatusWord()
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(!st)
            return nullptr;
        if(!st->status)
        {
            if(cudaMalloc(&st->status, 4 * sizeof(uint32_t)) != cudaSuccess
               || cudaMemset(st->status, 0, 4 * sizeof(uint32_t)) != cudaSuccess)
            {
                (void)cudaGetLastError();
                st->status = nullptr;
            }
        }
        return st->status;
    }

    int smCount()
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(!st)
            return 0;
        if(st->smCount == 0)
        {
            int dev = 0, n = 0;
            if(cudaGetDevice(&dev) == cudaSuccess
               && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess)
                st->smCount = n;
            else
                (void)cudaGetLastError();
        }
        return st->smCount;
    }

    void* deviceScratch(size_t bytes)
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(!st)
            return nullptr;
        if(st->scratchBytes < bytes)
        {
            if(st->scratch)
                (void)cudaFree(st->scratch);
            st->scratch      = nullptr;
            st->scratchBytes = 0;
            if(cudaMalloc(&st->scratch, bytes) != cudaSuccess)
            {
                (void)cudaGetLastError();
                return nullptr;
            }
            st->scratchBytes = bytes;
        }
        return st->scratch;
    }

    void* splitWorkspace(size_t bytes, uint32_t** counters)
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(!st || !counters)
            return nullptr;
        if(!st->splitCtr)
        {
            if(cudaMalloc(&st->splitCtr, 256 * sizeof(uint32_t)) != cudaSuccess
               || cudaMemset(st->splitCtr, 0, 256 * sizeof(uint32_t)) != cudaSuccess
               || cudaDeviceSynchronize() != cudaSuccess)
            {
                (void)cudaGetLastError();
                if(st->splitCtr)
                    (void)cudaFree(st->splitCtr);
                st->splitCtr = nullptr;
                return nullptr;
            }
        }
        if(st->splitWsBytes < bytes)
        {
            if(st->splitWs)
                (void)cudaFree(st->splitWs);
            st->splitWs      = nullptr;
            st->splitWsBytes = 0;
            if(cudaMalloc(&st->splitWs, bytes) != cudaSuccess)
            {
                (void)cudaGetLastError();
                return nullptr;
            }
            st->splitWsBytes = bytes;
        }
        *counters = st->splitCtr;
        return st->splitWs;
    }

    void* stagingBuffer(int slot, size_t bytes)
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(!st || slot < 0 || slot >= 4)
            return nullptr;
        if(st->stageBytes[slot] < bytes)
        {
            if(st->stage[slot])
                (void)cudaFree(st->stage[slot]);
            st->stage[slot]      = nullptr;
            st->stageBytes[slot] = 0;
            if(cudaMalloc(&st->stage[slot], bytes) != cudaSuccess)
            {
                (void)cudaGetLastError();
                return nullptr;
            }
            st->stageBytes[slot] = bytes;
        }
        return st->stage[slot];
    }

    unsigned int* launchCounter(cudaStream_t stream)
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(!st)
            return nullptr;
        if(!st->counters)
        {
            // zeroed once, before any launch can use them: the kernels put their counter back
            // to zero themselves
            if(cudaMalloc(&st->counters, 64 * 32) != cudaSuccess
               || cudaMemset(st->counters, 0, 64 * 32) != cudaSuccess
               || cudaDeviceSynchronize() != cudaSuccess)
            {
                (void)cudaGetLastError();
                if(st->counters)
                    (void)cudaFree(st->counters);
                st->counters = nullptr;
                return nullptr;
            }
        }
        // One counter per stream.  Launches of one stream run one after the other (a kernel
        // launched with programmatic stream serialization reads its counter only after
        // griddepcontrol.wait, i.e. after its predecessor has put the counter back to zero
        // and completed), so they can share a counter however many are queued; launches of
        // different streams may overlap and never share one.
        for(unsigned int i = 0; i < st->counterStreams; ++i)
            if(st->counterStream[i] == stream)
                return st->counters + i * 8u;
        if(st->counterStreams == 64u)
        {
            // A 65th stream: wait until every launch has finished (all counters are zero
            // again then) and start the table afresh.
            if(cudaDeviceSynchronize() != cudaSuccess)
            {
                (void)cudaGetLastError();
                return nullptr;
            }
            st->counterStreams = 0;
        }
        st->counterStream[st->counterStreams] = stream;
        return st->counters + (st->counterStreams++) * 8u;
    }

    void resetLaunchCounters()
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(st && st->counters && cudaMemset(st->counters, 0, 64 * 32) != cudaSuccess)
            (void)cudaGetLastError();
    }

    std::mutex* hostCallMutex()
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        return st ? &st->hostCall : nullptr;
    }

    HostPipe* hostPipe()
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        DeviceState*                st = current();
        if(!st)
            return nullptr;
        HostPipe& p = st->pipe;
        if(!p.ok)
        {
            bool good = cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking) == cudaSuccess
                        && cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking) == cudaSuccess
                        && cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming) == cudaSuccess
                        && cudaEventCreateWithFlags(&p.bReady, cudaEventDisableTiming)
                               == cudaSuccess;
            for(int i = 0; good && i < HOST_PIPE_MAX_CHUNKS; ++i)
                good = cudaEventCreateWithFlags(&p.in[i], cudaEventDisableTiming) == cudaSuccess
                       && cudaEventCreateWithFlags(&p.out[i], cudaEventDisableTiming)
                              == cudaSuccess;
            if(!good)
            {
                (void)cudaGetLastError();
                return nullptr;
            }
            p.ok = true;
        }
        return &p;
    }
} // namespace b200wmma

using namespace b200wmma;

extern "C" {

int b200wmma_version(void)
{
    return 10700; // tracks the rocWMMA API level 1.7.0 this library mirrors
}

const char* b200wmma_status_string(int status)
{
    switch(status)
    {
    case B200WMMA_OK:
        return "ok";
    case B200WMMA_ERR_INVALID_ARG:
        return "invalid argument";
    case B200WMMA_ERR_UNSUPPORTED:
        return "unsupported type, layout or shape";
    case B200WMMA_ERR_ALIGNMENT:
        return "pointer or leading dimension is not 16-byte aligned";
    case B200WMMA_ERR_CUDA:
        return "CUDA call failed (is a B200 visible?)";
    case B200WMMA_ERR_DEVICE_WAIT:
        return "a bounded wait inside a kernel ran out";
    case B200WMMA_ERR_TOO_LARGE:
        return "size beyond the documented maximum";
    }
    return "unknown status";
}

int b200wmma_check_device(void* stream, uint32_t* detail)
{
    B200WMMA_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    uint32_t* word = deviceStatusWord();
    if(!word)
        return B200WMMA_ERR_CUDA;
    uint32_t host[4] = {0, 0, 0, 0};
    B200WMMA_CUDA_TRY(cudaMemcpy(host, word, sizeof(host), cudaMemcpyDeviceToHost));
    if(detail)
        *detail = host[1];
    if(host[0] != 0)
    {
        B200WMMA_CUDA_TRY(cudaMemset(word, 0, sizeof(host)));
        // a kernel that gave up may have left its work counter in mid-count; the stream is
        // idle here, so put all of them back to zero
        B200WMMA_CUDA_TRY(cudaDeviceSynchronize());
        resetLaunchCounters();
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            DeviceState*                st = current();
            if(st && st->splitCtr
               && cudaMemset(st->splitCtr, 0, 256 * sizeof(uint32_t)) != cudaSuccess)
                (void)cudaGetLastError();
        }
        return B200WMMA_ERR_DEVICE_WAIT;
    }
    return B200WMMA_OK;
}

int b200wmma_shutdown(void)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    int                         prev = -1;
    (void)cudaGetDevice(&prev);
    for(int d = 0; d < MAX_DEVICES; ++d)
    {
        DeviceState& st = g_dev[d];
        bool any = st.status || st.scratch || st.stage[0] || st.stage[1] || st.stage[2]
                   || st.stage[3] || st.pipe.ok || st.counters || st.splitWs || st.splitCtr;
        if(!any)
            continue;
        if(cudaSetDevice(d) != cudaSuccess)
        {
            (void)cudaGetLastError();
            continue;
        }
        if(st.status)
            (void)cudaFree(st.status);
        if(st.scratch)
            (void)cudaFree(st.scratch);
        if(st.counters)
            (void)cudaFree(st.counters);
        if(st.splitWs)
            (void)cudaFree(st.splitWs);
        if(st.splitCtr)
            (void)cudaFree(st.splitCtr);
        st.splitWs      = nullptr;
        st.splitWsBytes = 0;
        st.splitCtr     = nullptr;
        for(void*& p : st.stage)
            if(p)
                (void)cudaFree(p);
        if(st.pipe.ok)
        {
            (void)cudaStreamDestroy(st.pipe.h2d);
            (void)cudaStreamDestroy(st.pipe.d2h);
            (void)cudaEventDestroy(st.pipe.start);
            (void)cudaEventDestroy(st.pipe.bReady);
            for(int i = 0; i < HOST_PIPE_MAX_CHUNKS; ++i)
            {
                (void)cudaEventDestroy(st.pipe.in[i]);
                (void)cudaEventDestroy(st.pipe.out[i]);
            }
        }
        st.status = nullptr;
        st.smCount = 0;
        st.scratch = nullptr;
        st.scratchBytes = 0;
        for(int i = 0; i < 4; ++i)
        {
            st.stage[i]      = nullptr;
            st.stageBytes[i] = 0;
        }
        st.pipe           = HostPipe{};
        st.counters       = nullptr;
        st.counterStreams = 0;
    }
    if(prev >= 0)
        (void)cudaSetDevice(prev);
    (void)cudaGetLastError();
    return B200WMMA_OK;
}
}
