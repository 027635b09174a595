// Bookkeeping for settings that CUDA keeps per DEVICE (cudaFuncSetAttribute, symbol addresses) while the
// code that applies them is shared by every context of the process: one flag per device index.
// Host-only, no CUDA dependency, so that it can be unit-tested without a GPU.
#pragma once

namespace mpq {

struct PerDeviceOnce {
    static constexpr int MAX_DEVICES = 64;
    bool done[MAX_DEVICES] = {};
    // true while the setting has not been applied on this device (always true for an index outside the
    // table: applying a per-device setting twice is harmless, skipping it is not)
    bool needs(int device) const { return device < 0 || device >= MAX_DEVICES || !done[device]; }
    void mark(int device)
    {
        if (device >= 0 && device < MAX_DEVICES) done[device] = true;
    }
};

}  // namespace mpq
