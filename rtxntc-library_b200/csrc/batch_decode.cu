// Decoding on several GPUs of one machine: a batch of texture sets, or one large set, is cut into
// work units (whole mips of a set, or bands of tile rows of its large mips), the units are handed out
// dynamically - largest first - to worker threads, each bound to one device, and every unit's texels
// are copied into the caller's host image of its set: the "final host gather".  The decode path has
// no exchange step, so the devices share nothing: no peer memory, no collective.
//
// The reference drives one device per context and has no multi-device code
// (include/libntc/ntc.h:1289-1290); this is the layer a client would otherwise write around it: one
// context per device, one host thread per context.
//
// A unit that fails on a device - its context cannot be created, a CUDA call fails, a bounded wait
// inside the decode kernel expires (NTCB_ERR_DEVICE_TIMEOUT) - goes back to the queue and is tried
// on another device; a device that keeps failing is retired.  The scheduling is independent of the
// GPU work: NtcbBatchOptions::worker replaces the latter, which is how the tests inject failing and
// slow workers on a machine without GPUs.

#include <cuda_runtime.h>

#include <algorithm>
#include <condition_variable>
#include <cstring>
#include <map>
#include <string>
#include <mutex>
#include <thread>
#include <vector>

#include "container.h"
#include "error.h"
#include "ntcb.h"

namespace ntcb
{
namespace
{

constexpr int kBandRows = 8;          // the decode kernels' tile height: no tile straddles two units
constexpr int kMinRowsPerBand = 64;   // a mip is only split into bands at least this tall
constexpr int kRetireAfterFailures = 2; // consecutive failed units after which a device is retired

struct MipSize
{
    int width, height;
};

// Cuts the items into units.  `target` texels per unit; an item of at most three quarters of a target
// stays whole (there are enough of them to balance the devices, and every unit of an item costs its
// worker a parse and an upload of the item's compressed data); one up to 1.5 targets becomes
// (mip 0) and (the other mips) - mip 0 is three quarters of a full chain - a larger one becomes
// `bands` units, each holding one band of tile rows of every mip tall enough to split; the mips too
// short to split go whole, largest first, to the unit with the least texels.
void PlanItem(int item, const NtcbTextureSetDesc& desc, uint64_t target, std::vector<NtcbBatchUnit>& units)
{
    std::vector<MipSize> mips(desc.mips);
    for (int m = 0; m < desc.mips; ++m)
        mips[m] = {std::max(desc.width >> m, 1), std::max(desc.height >> m, 1)};
    auto emptyUnit = [&]() {
        NtcbBatchUnit unit{};
        unit.item = item;
        unit.device = -1;
        return unit;
    };
    auto addRows = [&](NtcbBatchUnit& unit, int mip, int begin, int end) {
        unit.rowBegin[mip] = begin;
        unit.rowEnd[mip] = end;
        unit.texels += uint64_t(end - begin) * uint64_t(mips[mip].width);
    };

    const uint64_t total = desc.totalTexels;
    int bands = int(std::min<uint64_t>((total + target / 2) / std::max<uint64_t>(target, 1), 4096));
    bands = std::min(bands, std::max(mips[0].height / kMinRowsPerBand, 1));
    if (bands <= 1)
    {
        NtcbBatchUnit first = emptyUnit();
        addRows(first, 0, 0, mips[0].height);
        if (total * 4 <= target * 3)
        {
            for (int m = 1; m < desc.mips; ++m)
                addRows(first, m, 0, mips[m].height);
            units.push_back(first);
            return;
        }
        units.push_back(first);
        if (desc.mips > 1)
        {
            NtcbBatchUnit rest = emptyUnit();
            for (int m = 1; m < desc.mips; ++m)
                addRows(rest, m, 0, mips[m].height);
            units.push_back(rest);
        }
        return;
    }
    const size_t base = units.size();
    for (int b = 0; b < bands; ++b)
        units.push_back(emptyUnit());
    std::vector<int> whole;
    for (int m = 0; m < desc.mips; ++m)
    {
        if (mips[m].height < bands * kMinRowsPerBand)
        {
            whole.push_back(m);
            continue;
        }
        const int tileRows = (mips[m].height + kBandRows - 1) / kBandRows;
        for (int b = 0; b < bands; ++b)
        {
            const int begin = int(int64_t(tileRows) * b / bands) * kBandRows;
            const int end = std::min(mips[m].height, int(int64_t(tileRows) * (b + 1) / bands) * kBandRows);
            addRows(units[base + b], m, begin, end);
        }
    }
    std::sort(whole.begin(), whole.end(), [&](int a, int b) {
        return uint64_t(mips[a].width) * mips[a].height > uint64_t(mips[b].width) * mips[b].height;
    });
    for (int m : whole)
    {
        size_t least = base;
        for (size_t u = base; u < base + bands; ++u)
            if (units[u].texels < units[least].texels)
                least = u;
        addRows(units[least], m, 0, mips[m].height);
    }
}

int PlanUnits(const NtcbTextureSetDesc* descs, int numItems, int numDevices, int unitsPerDevice, std::vector<NtcbBatchUnit>& units)
{
    uint64_t total = 0;
    for (int i = 0; i < numItems; ++i)
    {
        const NtcbTextureSetDesc& d = descs[i];
        if (d.width < 1 || d.height < 1 || d.mips < 1 || d.mips > NTCB_MAX_MIPS)
        {
            SetError("Item %d has an invalid size (%d x %d) or mip count (%d).", i, d.width, d.height, d.mips);
            return NTCB_ERR_INVALID_ARGUMENT;
        }
        total += d.totalTexels;
    }
    const uint64_t target = std::max<uint64_t>(total / (uint64_t(numDevices) * uint64_t(unitsPerDevice)), 1);
    for (int i = 0; i < numItems; ++i)
        PlanItem(i, descs[i], target, units);
    // largest first: handed out in this order, the queue is a longest-processing-time-first schedule
    std::stable_sort(units.begin(), units.end(), [](const NtcbBatchUnit& a, const NtcbBatchUnit& b) { return a.texels > b.texels; });
    return NTCB_OK;
}

// ---------------------------------------------------------------------------------------------
// The queue
// ---------------------------------------------------------------------------------------------

struct Scheduler
{
    std::mutex mutex;
    std::condition_variable changed;
    std::vector<NtcbBatchUnit> units;
    std::vector<uint64_t> excluded;  // per unit: devices (by position in the device list) that failed it
    std::vector<int> state;          // per unit: 0 waiting, 1 running, 2 done, 3 failed for good
    std::vector<int> consecutiveFailures; // per device position
    uint64_t retired = 0;            // device positions that take no more work
    int open = 0;                    // units neither done nor failed for good
    int numDevices = 0;
    int maxAttempts = 3;

    // The next waiting unit this device may take (largest first), or -1 when there is none for it
    // right now; `finished` is set when no unit is open any more or this device is retired.
    int Take(int devicePosition, bool& finished)
    {
        std::unique_lock<std::mutex> lock(mutex);
        for (;;)
        {
            if (open == 0 || (retired >> devicePosition & 1))
            {
                finished = true;
                return -1;
            }
            for (size_t u = 0; u < units.size(); ++u)
            {
                if (state[u] == 0 && !(excluded[u] >> devicePosition & 1))
                {
                    state[u] = 1;
                    return int(u);
                }
            }
            // nothing for this device now: a unit that is running elsewhere may still come back
            changed.wait(lock);
        }
    }

    void Complete(int unit, int devicePosition, int device, int status)
    {
        std::lock_guard<std::mutex> lock(mutex);
        NtcbBatchUnit& u = units[unit];
        u.attempts += 1;
        u.device = device;
        u.status = status;
        if (status == NTCB_OK)
        {
            state[unit] = 2;
            consecutiveFailures[devicePosition] = 0;
            --open;
        }
        else
        {
            excluded[unit] |= uint64_t(1) << devicePosition;
            if (++consecutiveFailures[devicePosition] >= kRetireAfterFailures)
                retired |= uint64_t(1) << devicePosition;
            state[unit] = 0;
            if (u.attempts >= maxAttempts)
                Fail(unit);
        }
        Sweep();
        changed.notify_all();
    }

    void Retire(int devicePosition)
    {
        std::lock_guard<std::mutex> lock(mutex);
        retired |= uint64_t(1) << devicePosition;
        Sweep();
        changed.notify_all();
    }

private:
    void Fail(int unit)
    {
        if (state[unit] == 0)
        {
            state[unit] = 3;
            --open;
        }
    }

    // Waiting units that no live device may take any more are failed for good (otherwise the
    // workers would wait for them for ever).
    void Sweep()
    {
        const uint64_t all = numDevices >= 64 ? ~uint64_t(0) : (uint64_t(1) << numDevices) - 1;
        for (size_t u = 0; u < units.size(); ++u)
            if (state[u] == 0 && ((excluded[u] | retired) & all) == all)
                Fail(int(u));
    }
};

// ---------------------------------------------------------------------------------------------
// The GPU work of one worker thread
// ---------------------------------------------------------------------------------------------

struct DeviceWorker
{
    int device = 0;
    int numerics = NTCB_NUMERICS_REFERENCE;
    NtcbContext* context = nullptr;
    cudaStream_t copyStream = nullptr;
    // The worker's texture sets, one per SHAPE it has met: a unit of another item of the same dimensions
    // and latent shape is loaded into the buffers of the set that is already there (LoadFromMemory), so a
    // batch of equal sets allocates once per worker instead of once per item.
    struct Slot
    {
        NtcbTextureSet* set;
        NtcbTextureSetDesc desc;
        int item; // whose compressed data the set holds now
    };
    std::vector<Slot> slots;

    int Open()
    {
        int status = ntcb_context_create(device, &context);
        if (status != NTCB_OK)
            return status;
        cudaError_t err = cudaSetDevice(device);
        if (err == cudaSuccess)
            err = cudaStreamCreateWithFlags(&copyStream, cudaStreamNonBlocking);
        if (err != cudaSuccess)
            return CudaFailure("cudaStreamCreateWithFlags", err);
        return NTCB_OK;
    }

    void Close()
    {
        for (Slot& slot : slots)
            ntcb_texture_set_destroy(slot.set);
        slots.clear();
        if (copyStream)
        {
            cudaSetDevice(device);
            cudaStreamDestroy(copyStream);
            copyStream = nullptr;
        }
        if (context)
            ntcb_context_destroy(context);
        context = nullptr;
    }

    static bool SameShape(const NtcbTextureSetDesc& a, const NtcbTextureSetDesc& b)
    {
        return a.width == b.width && a.height == b.height && a.channels == b.channels && a.mips == b.mips
            && a.gridSizeScale == b.gridSizeScale && a.numFeatures == b.numFeatures;
    }

    // The texture set that holds (or now loads) the item's compressed data.
    int Acquire(const NtcbBatchItem& item, int itemIndex, const NtcbTextureSetDesc& itemDesc, NtcbTextureSet** outSet)
    {
        Slot* sameShape = nullptr;
        for (Slot& slot : slots)
        {
            if (slot.item == itemIndex)
            {
                *outSet = slot.set;
                return NTCB_OK;
            }
            if (!sameShape && SameShape(slot.desc, itemDesc))
                sameShape = &slot;
        }
        if (sameShape)
        {
            sameShape->item = -1;
            int status = ntcb_texture_set_load_from_memory(sameShape->set, item.container, item.containerBytes);
            if (status != NTCB_OK)
                return status;
            sameShape->item = itemIndex;
            *outSet = sameShape->set;
            return NTCB_OK;
        }
        NtcbTextureSetFeatures features{};
        features.outputLayout = NTCB_LAYOUT_INTERLEAVED;
        features.numerics = numerics;
        NtcbTextureSet* set = nullptr;
        int status = ntcb_texture_set_create_from_memory(context, item.container, item.containerBytes, &features, &set);
        if (status != NTCB_OK)
            return status;
        slots.push_back({set, itemDesc, itemIndex});
        *outSet = set;
        return NTCB_OK;
    }

    // Decodes the unit's rows and copies them into the item's host image (interleaved fp16, mip after mip).
    int Run(const NtcbBatchItem& item, const NtcbTextureSetDesc& itemDesc, const NtcbBatchUnit& unit)
    {
        NtcbTextureSet* set = nullptr;
        int acquired = Acquire(item, unit.item, itemDesc, &set);
        if (acquired != NTCB_OK)
            return acquired;
        const NtcbTextureSetDesc& desc = itemDesc;
        int status = NTCB_OK;
        if (item.hostTexelsBytes < size_t(desc.totalTexels) * size_t(desc.channels) * 2)
        {
            SetError("Item %d: the host image holds %zu bytes, the decoded set needs %zu.", unit.item, item.hostTexelsBytes,
                size_t(desc.totalTexels) * size_t(desc.channels) * 2);
            return NTCB_ERR_OUT_OF_RANGE;
        }
        int32_t ranges[2 * NTCB_MAX_MIPS] = {};
        for (int m = 0; m < desc.mips; ++m)
        {
            ranges[2 * m] = unit.rowBegin[m];
            ranges[2 * m + 1] = unit.rowEnd[m];
        }
        NtcbDecompressionStats stats{};
        status = ntcb_texture_set_decompress_rows(set, ranges, &stats, item.useInt8Weights); // waits; reports an expired wait
        if (status != NTCB_OK)
            return status;
        cudaError_t err = cudaSetDevice(device);
        if (err != cudaSuccess)
            return CudaFailure("cudaSetDevice", err);
        uint64_t mipOffset = 0; // texels of the mips before this one
        for (int m = 0; m < desc.mips; ++m)
        {
            const int width = std::max(desc.width >> m, 1), height = std::max(desc.height >> m, 1);
            if (unit.rowEnd[m] > unit.rowBegin[m])
            {
                void* deviceMip = nullptr;
                size_t mipBytes = 0;
                status = ntcb_texture_set_device_mip(set, m, &deviceMip, &mipBytes);
                if (status != NTCB_OK)
                    return status;
                const size_t rowBytes = size_t(width) * size_t(desc.channels) * 2;
                const size_t begin = size_t(unit.rowBegin[m]) * rowBytes, bytes = size_t(unit.rowEnd[m] - unit.rowBegin[m]) * rowBytes;
                err = cudaMemcpyAsync(static_cast<uint8_t*>(item.hostTexels) + mipOffset * size_t(desc.channels) * 2 + begin,
                    static_cast<const uint8_t*>(deviceMip) + begin, bytes, cudaMemcpyDeviceToHost, copyStream);
                if (err != cudaSuccess)
                    return CudaFailure("cudaMemcpyAsync (gather)", err);
            }
            mipOffset += uint64_t(width) * uint64_t(height);
        }
        err = cudaStreamSynchronize(copyStream);
        if (err != cudaSuccess)
            return CudaFailure("cudaStreamSynchronize (gather)", err);
        return NTCB_OK;
    }
};

// One run of a decoder: what the workers share while it lasts.
struct BatchJob
{
    NtcbBatchItem* items = nullptr;
    const NtcbTextureSetDesc* descs = nullptr;
    Scheduler scheduler;
};

} // namespace
} // namespace ntcb

// The threads of a batch decoder outlive its runs: a worker opens its context when the first run reaches it
// and keeps it, with the texture sets it has allocated, until the decoder is destroyed.
struct NtcbBatchDecoder
{
    std::vector<int> devices;
    NtcbBatchOptions options{};
    std::vector<std::thread> threads;
    std::mutex runMutex;  // one run at a time
    std::mutex mutex;     // guards what follows
    std::condition_variable wake, done;
    ntcb::BatchJob* job = nullptr;
    uint64_t generation = 0;
    int running = 0;
    bool closing = false;

    void WorkerLoop(int position)
    {
        using namespace ntcb;
        const int device = devices[size_t(position)];
        DeviceWorker worker;
        worker.device = device;
        worker.numerics = options.numerics;
        bool opened = false;
        uint64_t seen = 0;
        for (;;)
        {
            BatchJob* current = nullptr;
            {
                std::unique_lock<std::mutex> lock(mutex);
                wake.wait(lock, [&]() { return closing || generation != seen; });
                if (closing)
                    break;
                seen = generation;
                current = job;
            }
            if (!options.worker && !opened)
            {
                opened = worker.Open() == NTCB_OK; // tried again at the next run if it fails now
                if (!opened)
                    worker.Close();
            }
            Scheduler& scheduler = current->scheduler;
            if (!options.worker && !opened)
                scheduler.Retire(position);
            else
                for (;;)
                {
                    bool finished = false;
                    const int unit = scheduler.Take(position, finished);
                    if (finished)
                        break;
                    NtcbBatchUnit snapshot;
                    {
                        std::lock_guard<std::mutex> lock(scheduler.mutex);
                        snapshot = scheduler.units[size_t(unit)];
                    }
                    snapshot.device = device;
                    // (an exception - the host containers running out of memory - fails the unit like any other error)
                    const int result = Guarded("batch worker", [&]() {
                        return options.worker ? options.worker(options.workerUser, device, &snapshot)
                                              : worker.Run(current->items[snapshot.item], current->descs[snapshot.item], snapshot);
                    });
                    scheduler.Complete(unit, position, device, result);
                }
            {
                std::lock_guard<std::mutex> lock(mutex);
                if (--running == 0)
                    done.notify_all();
            }
        }
        worker.Close();
    }
};

extern "C"
{

int ntcb_plan_batch(const NtcbTextureSetDesc* descs, int numItems, int numDevices, int unitsPerDevice, NtcbBatchUnit* units,
    int maxUnits, int* outNumUnits)
{
    using namespace ntcb;
    if (!descs || numItems < 1 || numDevices < 1 || numDevices > 64 || !outNumUnits)
    {
        SetError("ntcb_plan_batch: needs items, 1..64 devices and outNumUnits.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    std::vector<NtcbBatchUnit> planned;
    int status = Guarded(__func__, [&]() { return PlanUnits(descs, numItems, numDevices, unitsPerDevice > 0 ? unitsPerDevice : 4, planned); });
    if (status != NTCB_OK)
        return status;
    *outNumUnits = int(planned.size());
    if (units)
    {
        if (int(planned.size()) > maxUnits)
        {
            SetError("ntcb_plan_batch: %zu units planned, room for %d.", planned.size(), maxUnits);
            return NTCB_ERR_OUT_OF_RANGE;
        }
        std::copy(planned.begin(), planned.end(), units);
    }
    ClearError();
    return NTCB_OK;
}

int ntcb_batch_decoder_create(const int* devices, int numDevices, const NtcbBatchOptions* options, NtcbBatchDecoder** outDecoder)
{
    using namespace ntcb;
    if (!outDecoder)
    {
        SetError("outDecoder is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    *outDecoder = nullptr;
    if (!devices || numDevices < 1 || numDevices > 64)
    {
        SetError("ntcb_batch_decoder_create: needs 1..64 devices.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    NtcbBatchOptions opt{};
    if (options)
        opt = *options;
    if (opt.maxAttempts < 1)
        opt.maxAttempts = 3;
    if (opt.unitsPerDevice < 1)
        opt.unitsPerDevice = 4;
    if (opt.workersPerDevice < 1)
        opt.workersPerDevice = opt.worker ? 1 : 2;
    if (opt.numerics != NTCB_NUMERICS_REFERENCE && opt.numerics != NTCB_NUMERICS_EXACT)
    {
        SetError("ntcb_batch_decoder_create: unknown numerics %d.", opt.numerics);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    NtcbBatchDecoder* decoder = nullptr;
    int status = Guarded(__func__, [&]() {
        decoder = new NtcbBatchDecoder;
        decoder->devices.assign(devices, devices + numDevices);
        decoder->options = opt;
        decoder->threads.reserve(size_t(numDevices) * size_t(opt.workersPerDevice));
        for (int position = 0; position < numDevices; ++position)
            for (int w = 0; w < opt.workersPerDevice; ++w)
                decoder->threads.emplace_back([decoder, position]() { decoder->WorkerLoop(position); });
        return NTCB_OK;
    });
    if (status != NTCB_OK)
    {
        // the threads that did start are told to leave and joined; the message of the failure stays
        ntcb_batch_decoder_destroy(decoder);
        return status;
    }
    *outDecoder = decoder;
    ClearError();
    return NTCB_OK;
}

void ntcb_batch_decoder_destroy(NtcbBatchDecoder* decoder)
{
    if (!decoder)
        return;
    {
        std::lock_guard<std::mutex> lock(decoder->mutex);
        decoder->closing = true;
    }
    decoder->wake.notify_all();
    for (std::thread& thread : decoder->threads)
        thread.join();
    delete decoder;
}

static int RunBatch(NtcbBatchDecoder* decoder, NtcbBatchItem* items, int numItems, NtcbBatchUnit* outUnits, int maxUnits,
    int* outNumUnits)
{
    using namespace ntcb;
    std::lock_guard<std::mutex> oneRunAtATime(decoder->runMutex);
    const NtcbBatchOptions& opt = decoder->options;
    const int numDevices = int(decoder->devices.size());

    // what each container holds (host only; every container is parsed and validated, on as many threads as
    // there are cores to spare: 64 containers of a megabyte each would otherwise cost the call 20 ms up front)
    std::vector<NtcbTextureSetDesc> descs(numItems);
    for (int i = 0; i < numItems; ++i)
    {
        items[i].status = NTCB_OK;
        if (!items[i].container || (!items[i].hostTexels && !opt.worker))
        {
            SetError("ntcb_decode_batch: item %d has no container or no host image.", i);
            return NTCB_ERR_INVALID_ARGUMENT;
        }
    }
    {
        const int probers = std::max(1, std::min<int>(numItems, std::min<unsigned>(std::thread::hardware_concurrency(), 16u)));
        std::vector<int> probeStatus(numItems, NTCB_OK);
        std::vector<std::string> probeMessage(numItems);
        std::vector<std::thread> pool;
        struct JoinAll // also when starting one of the threads throws
        {
            std::vector<std::thread>& threads;
            ~JoinAll()
            {
                for (std::thread& thread : threads)
                    if (thread.joinable())
                        thread.join();
            }
        };
        {
            JoinAll joinAll{pool};
            pool.reserve(size_t(probers));
            for (int t = 0; t < probers; ++t)
                pool.emplace_back([&, t]() {
                    for (int i = t; i < numItems; i += probers)
                    {
                        probeStatus[i] = ntcb_probe_container(items[i].container, items[i].containerBytes, &descs[i]);
                        if (probeStatus[i] != NTCB_OK)
                            (void)Guarded("ntcb_probe_container", [&]() {
                                probeMessage[i] = ntcb_last_error(); // the message is the probing thread's
                                return NTCB_OK;
                            });
                    }
                });
        }
        for (int i = 0; i < numItems; ++i)
            if (probeStatus[i] != NTCB_OK)
            {
                SetError("ntcb_decode_batch: item %d: %s", i, probeMessage[i].c_str());
                return probeStatus[i];
            }
    }

    BatchJob job;
    job.items = items;
    job.descs = descs.data();
    Scheduler& scheduler = job.scheduler;
    int status = PlanUnits(descs.data(), numItems, numDevices, opt.unitsPerDevice, scheduler.units);
    if (status != NTCB_OK)
        return status;
    const size_t count = scheduler.units.size();
    scheduler.excluded.assign(count, 0);
    scheduler.state.assign(count, 0);
    scheduler.consecutiveFailures.assign(numDevices, 0);
    scheduler.open = int(count);
    scheduler.numDevices = numDevices;
    scheduler.maxAttempts = opt.maxAttempts;

    {
        std::unique_lock<std::mutex> lock(decoder->mutex);
        decoder->job = &job;
        decoder->running = int(decoder->threads.size());
        ++decoder->generation;
        decoder->wake.notify_all();
        decoder->done.wait(lock, [&]() { return decoder->running == 0; });
        decoder->job = nullptr;
    }

    int failedUnits = 0;
    for (size_t u = 0; u < count; ++u)
    {
        const NtcbBatchUnit& unit = scheduler.units[u];
        if (scheduler.state[u] != 2)
        {
            ++failedUnits;
            if (items[unit.item].status == NTCB_OK)
                items[unit.item].status = unit.status != NTCB_OK ? unit.status : NTCB_ERR_CUDA;
        }
    }
    if (outNumUnits)
        *outNumUnits = int(count);
    if (outUnits)
        std::copy(scheduler.units.begin(), scheduler.units.begin() + std::min<size_t>(count, size_t(std::max(maxUnits, 0))), outUnits);
    if (failedUnits)
    {
        SetError("ntcb_decode_batch: %d of %zu work units could not be decoded on any device.", failedUnits, count);
        return NTCB_ERR_CUDA;
    }
    ClearError();
    return NTCB_OK;
}

int ntcb_batch_decoder_run(NtcbBatchDecoder* decoder, NtcbBatchItem* items, int numItems, NtcbBatchUnit* outUnits, int maxUnits,
    int* outNumUnits)
{
    using namespace ntcb;
    if (!decoder || !items || numItems < 1)
    {
        SetError("ntcb_batch_decoder_run: needs a decoder and items.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    // (the workers are handed the job only after everything that can throw here has been allocated)
    return Guarded(__func__, [&]() { return RunBatch(decoder, items, numItems, outUnits, maxUnits, outNumUnits); });
}

int ntcb_decode_batch(NtcbBatchItem* items, int numItems, const int* devices, int numDevices, const NtcbBatchOptions* options,
    NtcbBatchUnit* outUnits, int maxUnits, int* outNumUnits)
{
    using namespace ntcb;
    if (!items || numItems < 1 || !devices || numDevices < 1 || numDevices > 64)
    {
        SetError("ntcb_decode_batch: needs items and 1..64 devices.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (options && options->numerics != NTCB_NUMERICS_REFERENCE && options->numerics != NTCB_NUMERICS_EXACT)
    {
        SetError("ntcb_decode_batch: unknown numerics %d.", options->numerics);
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    NtcbBatchDecoder* decoder = nullptr;
    int status = ntcb_batch_decoder_create(devices, numDevices, options, &decoder);
    if (status != NTCB_OK)
        return status;
    status = ntcb_batch_decoder_run(decoder, items, numItems, outUnits, maxUnits, outNumUnits);
    // the message of a failed run must survive the teardown (ClearError is not called there)
    ntcb_batch_decoder_destroy(decoder);
    return status;
}

} // extern "C"
