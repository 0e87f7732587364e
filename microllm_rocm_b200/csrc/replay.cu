// Replay of a recorded list of launcher calls, with per-layer pointers swapped in.
//
// A step through a model of N structurally equal layers issues the same launches N times; only the
// layer's own tensors (weights, its pages of the cache) differ.  Issued one by one from Python, a call costs
// more host time (argument checks, ctypes marshalling) than a short kernel runs, so prompt portions of a
// few hundred tokens are bound by the host.  Instead the Python side records the calls of ONE layer (the
// launcher's address and its arguments as 64-bit slots, the floats apart), and this file issues them again
// for every other layer of the same structure: every pointer argument that equals one of the recorded
// layer's tensors is replaced by the same tensor of the layer being run.  One host call per layer, no
// interpreter between its launches.
//
// The launchers are the library's own exported functions (`int f(pointers, ints, long longs, floats...,
// stream)`), called through one generic function type.  That rests on the C calling convention of x86-64
// (System V) and AArch64 (AAPCS64): integer-class arguments travel in registers and then in 8-byte stack
// slots in order, floats in their own registers, independent of how the two kinds interleave; passing more
// slots than the callee reads is harmless because the caller owns the argument area.  Both are checked at
// compile time; on another ABI the engine keeps to its call-by-call path.
//
// The reference reaches the same goal by having its whole step function in C++
// (src/model/model.cpp:1448-1572: one packed host-to-device copy, then launches with no host work in between).
#include "common.cuh"

#if !defined(__x86_64__) && !defined(__aarch64__)
#error "replay.cu relies on the x86-64 System V or AArch64 procedure call standard"
#endif

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int MAX_INT_SLOTS = 28;
constexpr int MAX_FLOAT_SLOTS = 4;

}  // namespace

// One recorded call.  `slots`: the integer-class arguments (pointers, ints, long longs) in order, widened to
// 64 bits; `floats`: the float arguments in order; bit i of `pointer_mask` says that slot i is a pointer.
struct MlbCallRecord {
    void* function;
    unsigned long long slots[MAX_INT_SLOTS];
    float floats[MAX_FLOAT_SLOTS];
    unsigned int pointer_mask;
    int num_slots;
    int num_floats;
    int library;               // caller's tag for the shared object the function lives in (to read its error text)
};

typedef int (*GenericLauncher)(unsigned long long, unsigned long long, unsigned long long, unsigned long long,
                               unsigned long long, unsigned long long, unsigned long long, unsigned long long,
                               unsigned long long, unsigned long long, unsigned long long, unsigned long long,
                               unsigned long long, unsigned long long, unsigned long long, unsigned long long,
                               unsigned long long, unsigned long long, unsigned long long, unsigned long long,
                               unsigned long long, unsigned long long, unsigned long long, unsigned long long,
                               unsigned long long, unsigned long long, unsigned long long, unsigned long long,
                               float, float, float, float);

MLB_EXPORT int mlb_replay_record_bytes() { return (int)sizeof(MlbCallRecord); }
MLB_EXPORT int mlb_replay_max_slots() { return MAX_INT_SLOTS; }
MLB_EXPORT int mlb_replay_max_floats() { return MAX_FLOAT_SLOTS; }

// Issue `count` recorded calls in order.  `from[k]` -> `to[k]` (num_swaps pairs) replaces pointer arguments.
// Returns the first non-zero status a launcher gave (its index goes to *failed_at, and no further call is
// made), or 0.  *launched counts the calls made.
MLB_EXPORT int mlb_replay_calls(const MlbCallRecord* records, int count, const unsigned long long* from,
                                const unsigned long long* to, int num_swaps, int* failed_at, int* launched) {
    if (!records || count < 0 || num_swaps < 0 || (num_swaps > 0 && (!from || !to)))
        return fail(MLB_INVALID_ARGUMENT, "replay: bad arguments");
    if (failed_at) *failed_at = -1;
    int made = 0;
    for (int r = 0; r < count; ++r) {
        const MlbCallRecord& rec = records[r];
        if (!rec.function || rec.num_slots < 0 || rec.num_slots > MAX_INT_SLOTS || rec.num_floats < 0 || rec.num_floats > MAX_FLOAT_SLOTS) {
            if (failed_at) *failed_at = r;
            if (launched) *launched = made;
            return fail(MLB_INVALID_ARGUMENT, "replay: record %d is malformed", r);
        }
        unsigned long long a[MAX_INT_SLOTS];
        for (int i = 0; i < MAX_INT_SLOTS; ++i) a[i] = i < rec.num_slots ? rec.slots[i] : 0ull;
        for (int i = 0; i < rec.num_slots; ++i) {
            if (!((rec.pointer_mask >> i) & 1u) || a[i] == 0ull) continue;
            for (int k = 0; k < num_swaps; ++k)
                if (a[i] == from[k]) { a[i] = to[k]; break; }
        }
        const float* f = rec.floats;
        const int status = ((GenericLauncher)rec.function)(
            a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], a[9], a[10], a[11], a[12], a[13], a[14], a[15], a[16],
            a[17], a[18], a[19], a[20], a[21], a[22], a[23], a[24], a[25], a[26], a[27], f[0], f[1], f[2], f[3]);
        ++made;
        if (status != 0) {
            if (failed_at) *failed_at = r;
            if (launched) *launched = made;
            return status;
        }
    }
    if (launched) *launched = made;
    return MLB_OK;
}

// A launcher-shaped function without a kernel, for checking the generic call on the host: ten integer-class
// arguments (so that some travel on the stack) interleaved with two floats.  It writes what it received.
MLB_EXPORT int mlb_replay_probe(const void* p0, long long a1, int a2, float f0, void* p3, int a4, int a5, int a6,
                                long long a7, float f1, int a8, long long* out) {
    if (!out) return fail(MLB_INVALID_ARGUMENT, "replay probe: no output");
    out[0] = (long long)(uintptr_t)p0; out[1] = a1; out[2] = a2; out[3] = (long long)(uintptr_t)p3; out[4] = a4;
    out[5] = a5; out[6] = a6; out[7] = a7; out[8] = a8;
    out[9] = (long long)(f0 * 1000.0f); out[10] = (long long)(f1 * 1000.0f);
    if (a2 < 0) return fail(MLB_INVALID_ARGUMENT, "replay probe: refused on purpose (a2 = %d)", a2);
    return MLB_OK;
}
