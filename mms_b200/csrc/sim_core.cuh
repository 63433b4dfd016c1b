// sim_core.cuh — per-lane simulator state and the per-request step.
//
// One THREAD simulates one stream of requests for one candidate placement
// (alpa_serve/simulator/controller.py:579-622 is the loop body restated in
// sim_step below).  Mutable state (the stage clocks) lives in shared
// memory as [entry][lane], so lane-private accesses fall on distinct banks;
// shared memory is what limits the number of resident warps, so the
// read-only replica lists stay in global memory (a 16-byte row per model with
// its first four replicas, fetched two requests ahead, and a second one with
// the next four, fetched one request ahead where the first is full; served by
// L2).  Everything is addressed by
// 32-bit element offsets into the block's one dynamic shared array, which
// keeps the accesses plain LDS/STS with immediate offsets.  The dependent
// chain per request is kept short: trace values are fetched three requests
// ahead and the replica row two requests ahead (neither depends on simulator
// state), the clocks of up to 4 replicas and of up to 8 pipeline stages are
// loaded together, and the max/add chain runs in registers.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "mms_sim.h"

namespace mms {

constexpr double kInf = 1e100;          // alpa_serve/util.py:23
constexpr double kOverhead = 0.011;     // controller.py:575
constexpr int kLanes = 32;              // streams per warp
constexpr int kMaxBlockWarps = 12;      // warps of a stream-kernel block
constexpr int kMaxWarpsPerSm = 12;      // the stream kernel's registers allow that many
constexpr int kClockPad = 8;            // readable slots past the last clock
constexpr int kRowWords = 4;            // u32 words of a model's replica row

extern __shared__ __align__(16) unsigned char smem[];

#define SM_F64(i) (reinterpret_cast<double *>(smem)[(i)])
#define SM_U32(i) (reinterpret_cast<uint32_t *>(smem)[(i)])
#define SM_U16(i) (reinterpret_cast<uint16_t *>(smem)[(i)])
#define SM_F32(i) (reinterpret_cast<float *>(smem)[(i)])

// On-chip replica entry: group | LAST clock slot << 8 | stages << 16 | column << 24.
// (The caller's model_rep carries the FIRST slot; setup converts.)
__device__ __forceinline__ uint32_t rep_group(uint32_t e) { return e & 0xFFu; }
__device__ __forceinline__ uint32_t rep_last(uint32_t e) { return (e >> 8) & 0xFFu; }
__device__ __forceinline__ uint32_t rep_stages(uint32_t e) { return (e >> 16) & 0xFFu; }
__device__ __forceinline__ uint32_t rep_column(uint32_t e) { return e >> 24; }

// Shared memory of a block: the latency table shared by all its warps, then
// one region per warp with that warp's 32 lane-private states.
struct SmemLayout {
    size_t latency;                      // from the start of the array
    size_t warp0, warp_bytes;            // first warp's region; size of a region
    size_t clocks, stage_tmp;            // inside a warp's region
    size_t total;                        // bytes of a one-warp block
    int tmp_stages;
};

// lat_elems: entries of the shared latency table kept on chip (0 = read it
// from global memory), as f32 or, with lat_f64, widened to f64.  Counters are not kept on chip: the step records
// its decision per request (see Lane::dec) and count_kernel tallies them.
__host__ __device__ inline SmemLayout smem_layout(int M, int G, int /*P*/, int T, int S,
                                                  bool group_good, int lat_elems,
                                                  bool lat_f64 = false)
{
    SmemLayout L;
    L.latency = 0;
    L.warp0 = ((lat_f64 ? sizeof(double) : sizeof(float)) * (size_t)((lat_elems + 3) & ~3) + 15) &
              ~(size_t)15;
    size_t off = 0;
    L.clocks = off;     off += sizeof(double) * (size_t)(T + kClockPad) * kLanes;
    L.tmp_stages = S > 8 ? S - 8 : 0;
    L.stage_tmp = off;  off += sizeof(double) * (size_t)L.tmp_stages * kLanes;
    L.warp_bytes = (off + 15) & ~(size_t)15;
    L.total = L.warp0 + L.warp_bytes;
    return L;
}

// A lane's view of its state: element offsets into the typed views of the
// shared array, already including the lane; entries are kLanes apart.
struct Lane {
    uint32_t clk;             // f64 index of clock slot 0
    uint32_t tmp;             // f64 index, stages beyond the 8th of a deep pipeline
    uint32_t lat_sm;          // f32 index of the on-chip latency table
    void *dec;                // element (request 0, this candidate) of the decision array: per request
                              //   0 = not dispatched, else (group + 1) | accepted << 7 in a
                              //   byte (up to 126 groups), or | accepted << 15 in 16 bits
    uint32_t dec_pitch;       // elements between consecutive requests in that array
    bool dec_wide;            // 16-bit decisions
    uint32_t dec_word;        // byte decisions: the records of up to four consecutive requests,
                              //   gathered here and stored as one 32-bit word behind every fourth
                              //   request (recorded stretches begin at multiples of 4)
    const uint4 *rows;        // [M + 1] replica rows of this candidate (global memory,
                              //   kLanes apart: the rows of 32 consecutive candidates for one
                              //   model are contiguous, so a warp fetches them coalesced): the
                              //   model's first four replicas, kNoReplica where it has fewer;
                              //   row M is empty (unknown models)
    const uint4 *rows_b;      // the same for replicas five to eight; a model with more than
                              //   eight has kMoreReplicas in word 3 of this row (the full list
                              //   is then read from the caller's tables)
    const uint32_t *rep_raw;  // the caller's model_rep row of this candidate
    const uint16_t *rep_off;  // the caller's model_off row of this candidate
    const float *lat_gl;      // this candidate's table in global memory
    bool lat_on_chip;
    bool lat_f64;             // on chip as doubles
    int32_t M, C, S;
    uint32_t status;
    uint32_t staging;         // byte offset of the warp's decoded-request records (kStagedBytes),
                              //   for the step that decodes ahead (staged_step); 0 = none
};

// Row words that are not replicas.  Both address clock slot 0 / one stage /
// latency column 0, so that the branch-free step can load through them.
constexpr uint32_t kNoReplica = 0xFF010000u;
constexpr uint32_t kMoreReplicas = 0xFE010000u;

// Requests in flight.  Request i is ready to execute: its replica row is in
// registers, and so is the row of request i+1.  While i executes, the row of
// request i+2 and the trace values of request i+3 are fetched, so every
// global load has a whole step or more to arrive; so is the second row of
// request i+1, by the lanes whose first row of it is full.  Nothing fetched
// ahead depends on simulator state.
struct Pipe {
    double ts; float slo; int32_t m; uint4 r;
    uint4 rb;                 // replicas five to eight of request i (kNoReplica: none)
    double ts1; float slo1; int32_t m1; uint4 r1;
    double ts2; float slo2; int32_t m2;
    const double *arrivals; const int32_t *model_ids; const float *slos;   // request 0 of this lane's trace
    uint32_t pitch;           // elements between consecutive requests of the trace
    int32_t last;             // highest readable request index
};

__device__ __forceinline__ int32_t clean_model(Lane &ln, int32_t m)
{
    if (m >= ln.M) { ln.status |= MMS_STATUS_BAD_INDEX; return -1; }
    return m;
}

__device__ __forceinline__ uint4 fetch_row(const Lane &ln, int32_t m)
{
    return __ldg(ln.rows + (m < 0 ? ln.M : m) * kLanes);
}

// The second row of model m, given its first: only a full first row has one.
__device__ __forceinline__ uint4 fetch_row_b(const Lane &ln, int32_t m, const uint4 &first)
{
    if (first.w >= kMoreReplicas) return make_uint4(kNoReplica, kNoReplica, kNoReplica, kNoReplica);
    return __ldg(ln.rows_b + (m < 0 ? ln.M : m) * kLanes);
}

// Fills the pipe so that request `i` is ready to execute.
__device__ __forceinline__ void pipe_prime(Lane &ln, Pipe &p, int32_t i)
{
    const int32_t i0 = i < p.last ? i : p.last;
    const int32_t i1 = i + 1 < p.last ? i + 1 : p.last;
    const int32_t i2 = i + 2 < p.last ? i + 2 : p.last;
    const size_t o0 = (size_t)i0 * p.pitch, o1 = (size_t)i1 * p.pitch, o2 = (size_t)i2 * p.pitch;
    p.ts = __ldg(p.arrivals + o0); p.slo = __ldg(p.slos + o0);
    p.m = clean_model(ln, __ldg(p.model_ids + o0));
    p.ts1 = __ldg(p.arrivals + o1); p.slo1 = __ldg(p.slos + o1);
    p.m1 = clean_model(ln, __ldg(p.model_ids + o1));
    p.ts2 = __ldg(p.arrivals + o2); p.slo2 = __ldg(p.slos + o2);
    p.m2 = __ldg(p.model_ids + o2);            // checked by the step that fetches its row
    p.r = fetch_row(ln, p.m);
    p.r1 = fetch_row(ln, p.m1);
    p.rb = fetch_row_b(ln, p.m, p.r);
}

// max of two times.  Times are never NaN (arrivals are checked to be finite,
// latencies are finite or +inf), so one compare and a select do.
__device__ __forceinline__ double tmax(double a, double b) { return a > b ? a : b; }

// Latency table entry `at` (model, column, stage flattened), widened.
__device__ __forceinline__ double lat_at(const Lane &ln, uint32_t at)
{
    if (!ln.lat_on_chip) return (double)__ldg(ln.lat_gl + at);
    return ln.lat_f64 ? SM_F64(ln.lat_sm + at) : (double)SM_F32(ln.lat_sm + at);
}

// Replica entry as the caller gives it (first clock slot) -> with the LAST slot.
__device__ __forceinline__ uint32_t rep_to_last(uint32_t e)
{
    const uint32_t ns = (e >> 16) & 0xFFu, first = (e >> 8) & 0xFFu;
    return (e & 0xFFFF00FFu) | (((first + ns - 1) & 0xFFu) << 8);
}

// Executes request `i` (controller.py:579-622, or :519-555 with kLegacy) and
// advances the pipe.  Returns finish - arrival, which is 0.0 for a dropped
// request (the reference stores finish = arrival for those).
//   record  write the decision and the per-request outputs (off during run-in)
// The common path has no divergent branch: a lane whose candidate has no
// replica of the model, or drops the request, runs the same instructions on
// harmless addresses and its stores are predicated off.  The step is large;
// callers keep a single call site per kernel so that the hot loop stays
// inside the instruction cache.
//   kNarrow  for a warp in which ONE lane works (the serial repairs): real
//            branches, so that only the replicas and the stages that exist are
//            touched — about a quarter fewer instructions, and no other lane to hold up.
//   kSlim    (with kNarrow) what the caller checked once is known at compile
//            time here: the latency table is on chip as doubles and decisions
//            are bytes.  The pipelines of 1, 2, 4 and 8 stages — every power-
//            of-two partition of a node — then run as straight-line code (all
//            loads first, one chain, the stores), without a test per stage.
template <bool kFull, bool kGroupGood, bool kLegacy, bool kNarrow = false, bool kSlim = false>
__device__ __forceinline__ double sim_step(Lane &ln, Pipe &p, int32_t i, bool record,
                                           double *finish_out, uint8_t *good_out)
{
    static_assert(!kSlim || (kNarrow && !kLegacy && !kFull), "kSlim is a form of the narrow step");
    const double ts = p.ts;
    const float slo_f = p.slo;
    const int32_t m = p.m;
    const uint32_t e0 = p.r.x, e1 = p.r.y, e2 = p.r.z, e3 = p.r.w;

    // ---- state-independent fetches for the requests behind this one -------
    // the model id fetched a step ago is looked at only now, a whole step after its load
    // was issued (checking it when it is fetched would make every step wait for that load)
    p.m2 = clean_model(ln, p.m2);
    const uint4 r2 = fetch_row(ln, p.m2);
    const uint4 rb1 = fetch_row_b(ln, p.m1, p.r1);
    const size_t i3 = (size_t)(i + 3 < p.last ? i + 3 : p.last) * p.pitch;
    const double ts3 = __ldg(p.arrivals + i3);
    const float slo3 = __ldg(p.slos + i3);
    const int32_t m3raw = __ldg(p.model_ids + i3);

    // ---- :589-598 replica whose last-stage clock is strictly smallest ------
    double best = kInf;
    uint32_t pick = 0x00010000u;          // group 0, slot 0, one stage, column 0
    if constexpr (kNarrow) {
        // a row is filled from word 0 on
        if (e0 < kMoreReplicas) {
            best = SM_F64(ln.clk + rep_last(e0) * kLanes);
            pick = e0;
            if (!(best < kInf)) { best = kInf; pick = 0x00010000u; }
            if (e1 < kMoreReplicas) {
                const double c1 = SM_F64(ln.clk + rep_last(e1) * kLanes);
                if (c1 < best) { best = c1; pick = e1; }
                if (e2 < kMoreReplicas) {
                    const double c2 = SM_F64(ln.clk + rep_last(e2) * kLanes);
                    if (c2 < best) { best = c2; pick = e2; }
                    if (e3 < kMoreReplicas) {
                        const double c3 = SM_F64(ln.clk + rep_last(e3) * kLanes);
                        if (c3 < best) { best = c3; pick = e3; }
                    }
                }
            }
        }
    } else {
        const double c0 = SM_F64(ln.clk + rep_last(e0) * kLanes);
        const double c1 = SM_F64(ln.clk + rep_last(e1) * kLanes);
        const double c2 = SM_F64(ln.clk + rep_last(e2) * kLanes);
        const double c3 = SM_F64(ln.clk + rep_last(e3) * kLanes);
        if (e0 < kMoreReplicas && c0 < best) { best = c0; pick = e0; }
        if (e1 < kMoreReplicas && c1 < best) { best = c1; pick = e1; }
        if (e2 < kMoreReplicas && c2 < best) { best = c2; pick = e2; }
        if (e3 < kMoreReplicas && c3 < best) { best = c3; pick = e3; }
    }
    if (p.rb.x < kMoreReplicas) {         // five replicas or more: the second row
        const uint32_t e4 = p.rb.x, e5 = p.rb.y, e6 = p.rb.z, e7 = p.rb.w;
        const double c4 = SM_F64(ln.clk + rep_last(e4) * kLanes);
        const double c5 = SM_F64(ln.clk + rep_last(e5) * kLanes);
        const double c6 = SM_F64(ln.clk + rep_last(e6) * kLanes);
        const double c7 = SM_F64(ln.clk + rep_last(e7) * kLanes);
        if (c4 < best) { best = c4; pick = e4; }
        if (e5 < kMoreReplicas && c5 < best) { best = c5; pick = e5; }
        if (e6 < kMoreReplicas && c6 < best) { best = c6; pick = e6; }
        if (e7 < kMoreReplicas && c7 < best) { best = c7; pick = e7; }
        if (e7 == kMoreReplicas) {        // rare: the whole list, from the caller's tables
            const uint32_t lo = ln.rep_off[m], hi = ln.rep_off[m + 1];
            best = kInf;
            pick = 0x00010000u;
            for (uint32_t r = lo; r < hi; ++r) {
                const uint32_t e = rep_to_last(__ldg(ln.rep_raw + r));
                const double c = SM_F64(ln.clk + rep_last(e) * kLanes);
                if (c < best) { best = c; pick = e; }
            }
        }
    }
    const bool found = best < kInf;

    const uint32_t g = rep_group(pick);
    const uint32_t ns = kLegacy ? 1u : rep_stages(pick);
    const uint32_t ck = ln.clk + (rep_last(pick) + 1 - ns) * kLanes;   // first slot
    const uint32_t row = ((uint32_t)(m < 0 ? 0 : m) * ln.C + rep_column(pick)) * ln.S;
    double f;
    double t0, t1 = 0, t2 = 0, t3 = 0, t4 = 0, t5 = 0, t6 = 0, t7 = 0;
    (void)t2; (void)t3; (void)t4; (void)t5; (void)t6; (void)t7;
    bool slim_done = false;          // kSlim: the chain, the test and the stores are through
    bool slim_accept = false;
    if constexpr (kSlim) {
        const uint32_t lr = ln.lat_sm + row;             // the table holds doubles
        auto run = [&](auto depth) {
            constexpr int kDepth = decltype(depth)::value;
            double k[kDepth], l[kDepth], t[kDepth];
#pragma unroll
            for (int s = 0; s < kDepth; ++s) {
                k[s] = SM_F64(ck + s * kLanes);
                l[s] = SM_F64(lr + s);
            }
            double cur = ts;
#pragma unroll
            for (int s = 0; s < kDepth; ++s) {           // :605-608
                cur = tmax(cur, k[s]) + l[s];
                t[s] = cur;
            }
            f = cur + kOverhead;                         // :610
            slim_accept = found && (f - ts <= (double)slo_f);     // :613
            if (slim_accept) {
#pragma unroll
                for (int s = 0; s < kDepth; ++s) SM_F64(ck + s * kLanes) = t[s];
            }
            slim_done = true;
        };
        switch (ns) {
            case 1: run(std::integral_constant<int, 1>{}); break;
            case 2: run(std::integral_constant<int, 2>{}); break;
            case 4: run(std::integral_constant<int, 4>{}); break;
            case 8: run(std::integral_constant<int, 8>{}); break;
            default: break;                              // other depths: the general code below
        }
    }
    if (slim_done) {
        t0 = 0;
    } else if constexpr (kNarrow && !kLegacy) {
        // :605-610 stage by stage, as far as the group has stages
        auto lat = [&](uint32_t k) { return lat_at(ln, row + k); };
        t0 = tmax(ts, SM_F64(ck)) + lat(0);
        double t = t0;
        if (ns > 1) {
            t1 = tmax(t0, SM_F64(ck + kLanes)) + lat(1); t = t1;
            if (ns > 2) {
                t2 = tmax(t1, SM_F64(ck + 2 * kLanes)) + lat(2); t = t2;
                if (ns > 3) {
                    t3 = tmax(t2, SM_F64(ck + 3 * kLanes)) + lat(3); t = t3;
                    if (ns > 4) {
                        t4 = tmax(t3, SM_F64(ck + 4 * kLanes)) + lat(4); t = t4;
                        if (ns > 5) {
                            t5 = tmax(t4, SM_F64(ck + 5 * kLanes)) + lat(5); t = t5;
                            if (ns > 6) {
                                t6 = tmax(t5, SM_F64(ck + 6 * kLanes)) + lat(6); t = t6;
                                if (ns > 7) {
                                    t7 = tmax(t6, SM_F64(ck + 7 * kLanes)) + lat(7); t = t7;
                                    for (uint32_t k = 8; k < ns; ++k) {
                                        t = tmax(t, SM_F64(ck + k * kLanes)) + lat(k);
                                        SM_F64(ln.tmp + (k - 8) * kLanes) = t;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
        f = t + kOverhead;                               // :610
    } else {
        // all stage clocks and latencies are fetched at once; the max/add chain
        // then runs in registers
        const double k0 = SM_F64(ck), k1 = SM_F64(ck + kLanes), k2 = SM_F64(ck + 2 * kLanes),
                     k3 = SM_F64(ck + 3 * kLanes), k4 = SM_F64(ck + 4 * kLanes),
                     k5 = SM_F64(ck + 5 * kLanes), k6 = SM_F64(ck + 6 * kLanes),
                     k7 = SM_F64(ck + 7 * kLanes);
        double l0, l1, l2 = 0, l3 = 0, l4 = 0, l5 = 0, l6 = 0, l7 = 0;
        if (ln.lat_on_chip && ln.lat_f64) {
            const uint32_t lr = ln.lat_sm + row;
            l0 = SM_F64(lr); l1 = SM_F64(lr + 1); l2 = SM_F64(lr + 2); l3 = SM_F64(lr + 3);
            l4 = SM_F64(lr + 4); l5 = SM_F64(lr + 5); l6 = SM_F64(lr + 6); l7 = SM_F64(lr + 7);
        } else if (ln.lat_on_chip) {
            // rows are padded so that 8 entries are always readable
            const uint32_t lr = ln.lat_sm + row;
            l0 = (double)SM_F32(lr); l1 = (double)SM_F32(lr + 1);
            l2 = (double)SM_F32(lr + 2); l3 = (double)SM_F32(lr + 3);
            l4 = (double)SM_F32(lr + 4); l5 = (double)SM_F32(lr + 5);
            l6 = (double)SM_F32(lr + 6); l7 = (double)SM_F32(lr + 7);
        } else {
            const float *lat = ln.lat_gl + row;
            const int sm = ln.S - 1;   // clamp reads to the table row
            l0 = (double)__ldg(lat); l1 = (double)__ldg(lat + (1 < sm ? 1 : sm));
            if (ns > 2) {
                l2 = (double)__ldg(lat + (2 < sm ? 2 : sm));
                l3 = (double)__ldg(lat + (3 < sm ? 3 : sm));
                l4 = (double)__ldg(lat + (4 < sm ? 4 : sm));
                l5 = (double)__ldg(lat + (5 < sm ? 5 : sm));
                l6 = (double)__ldg(lat + (6 < sm ? 6 : sm));
                l7 = (double)__ldg(lat + (7 < sm ? 7 : sm));
            }
        }
        if (kLegacy) {
            // :543-544 one clock per group; latency row = {sum, max}
            const double start = tmax(k0, ts);
            f = start + l0 + kOverhead;
            t0 = start + l1;
        } else {
            // :605-610, written without branches: stages past the group's last one
            // are computed and thrown away
            // the chain runs through all eight slots; the finish time is picked from the
            // group's last stage afterwards, so that no select sits between two stages
            t0 = tmax(ts, k0) + l0;
            t1 = tmax(t0, k1) + l1;
            t2 = tmax(t1, k2) + l2;
            t3 = tmax(t2, k3) + l3;
            t4 = tmax(t3, k4) + l4;
            t5 = tmax(t4, k5) + l5;
            t6 = tmax(t5, k6) + l6;
            t7 = tmax(t6, k7) + l7;
            const uint32_t d = ns - 1;
            const double ta = (d & 1) ? t1 : t0, tb = (d & 1) ? t3 : t2;
            const double tc = (d & 1) ? t5 : t4, td = (d & 1) ? t7 : t6;
            const double te = (d & 2) ? tb : ta, tf = (d & 2) ? td : tc;
            double t = (d & 4) ? tf : te;
            if (ns > 8) {
                t = t7;
                for (uint32_t k = 8; k < ns; ++k) {
                    const double lk = lat_at(ln, row + k);
                    t = tmax(t, SM_F64(ck + k * kLanes)) + lk;
                    SM_F64(ln.tmp + (k - 8) * kLanes) = t;
                }
            }
            f = t + kOverhead;                               // :610
        }
    }
    const bool accept = slim_done ? slim_accept : (found && (f - ts <= (double)slo_f));   // :613-619
    const double fin = accept ? f : ts;
    if (accept && !slim_done) {
        SM_F64(ck) = t0;
        if (ns > 1) SM_F64(ck + kLanes) = t1;
        if (ns > 2) SM_F64(ck + 2 * kLanes) = t2;
        if (ns > 3) SM_F64(ck + 3 * kLanes) = t3;
        if (ns > 4) SM_F64(ck + 4 * kLanes) = t4;
        if (ns > 5) SM_F64(ck + 5 * kLanes) = t5;
        if (ns > 6) SM_F64(ck + 6 * kLanes) = t6;
        if (ns > 7) SM_F64(ck + 7 * kLanes) = t7;
        if (ns > 8)
            for (uint32_t k = 8; k < ns; ++k)
                SM_F64(ck + k * kLanes) = SM_F64(ln.tmp + (k - 8) * kLanes);
    }
    if (record) {   // :611, :617-618 are tallied from this record by count_kernel
        // four consecutive requests of a candidate sit side by side (count_kernel reads them
        // with one load): element (i, b) is at ((i / 4) * pitch + b) * 4 + i % 4
        if (!kSlim && ln.dec_wide) {
            const size_t at = ((size_t)(i >> 2) * ln.dec_pitch) * 4 + (size_t)(i & 3);
            static_cast<uint16_t *>(ln.dec)[at] =
                (uint16_t)(found ? (g + 1u) | (accept ? 0x8000u : 0u) : 0u);
        } else {
            // one 32-bit store per four requests instead of four byte stores: a quarter
            // of the store instructions, and every sector a warp writes is written whole
            const uint32_t rec = found ? (g + 1u) | (accept ? 0x80u : 0u) : 0u;
            ln.dec_word |= rec << (8 * (i & 3));
            if ((i & 3) == 3 || i == p.last) {
                static_cast<uint32_t *>(ln.dec)[(size_t)(i >> 2) * ln.dec_pitch] = ln.dec_word;
                ln.dec_word = 0;
            }
        }
    }
    if (kFull && record) {
        finish_out[i] = fin;
        good_out[i] = accept ? 1 : 0;
    }

    // ---- advance the pipe ---------------------------------------------------
    p.ts = p.ts1; p.slo = p.slo1; p.m = p.m1; p.r = p.r1; p.rb = rb1;
    p.ts1 = p.ts2; p.slo1 = p.slo2; p.m1 = p.m2; p.r1 = r2;
    p.ts2 = ts3; p.slo2 = slo3; p.m2 = m3raw;      // unchecked until the next step fetches its row
    return fin - ts;
}

// ---- the one-lane step with the warp decoding ahead ---------------------------
//
// Serial repairs, the chain kernel and every sweep over an overloaded placement
// walk ONE dependent chain per warp, and most of what sim_step executes per
// request there does not depend on the simulator's state: fetching the trace,
// the model's replica row, turning its entries into clock and latency
// addresses.  Here the 32 lanes of the warp do that part for 32 consecutive
// requests at once (staged_decode: one record per request in shared memory),
// and the recurrence then runs over the records (staged_step: replica choice,
// max/add chain, SLO test, clock stores, decision record) with less than half
// the instructions per request.  Every lane executes the recurrence, on the
// same addresses with the same values (the caller sets all lanes up as lane 0):
// a warp issues one instruction for 32 lanes or for one at the same cost, and
// control flow that is the same in every lane needs no lane to wait for
// another.  Needs what the slim step needs (table on chip as doubles, byte
// decisions), models with at most eight replicas, and every shared-memory index
// below 65536.
constexpr int kStageAhead = 32;
constexpr size_t kStagedBytes = (size_t)kStageAhead * (4 * 16 + 8 + 8);

// A request's record: 80 bytes — uint4 a, b, a2, b2 and two doubles:
//   a, a2   per replica (first four, next four): f64 index of its last-stage clock |
//           f64 index of its first clock << 16; 0xFFFFFFFF = no replica
//   b, b2   per replica: f64 index of its latency row | stages << 16 | group << 24
//   ts, slo arrival time and SLO (widened)
constexpr uint32_t kRecordBytes = 80;
static_assert(kStagedBytes == kStageAhead * kRecordBytes, "record size");

struct Staged {
    uint32_t rec;             // byte offset of record 0
    int32_t base;             // requests [base, base + kStageAhead) are decoded
    int32_t next;             // the request whose record is in the registers below
    uint4 a, b;
    double ts, slo;
    // this lane's trace element of the block behind the decoded one, loaded while that one is
    // worked through (a block of steps is ample time for the loads to arrive)
    int32_t ahead_base;
    double ahead_ts;
    float ahead_slo;
    int32_t ahead_m;          // unchecked
};

__device__ __forceinline__ Staged staged_init(const Lane &ln)
{
    Staged st;
    st.rec = ln.staging;
    st.base = -0x40000000;
    st.next = -1;
    st.a = st.b = make_uint4(0, 0, 0, 0);
    st.ts = st.slo = 0.0;
    st.ahead_base = -0x40000000;
    st.ahead_ts = 0.0; st.ahead_slo = 0.0f; st.ahead_m = -1;
    return st;
}

// The record's first half and its times; the second half (replicas five to eight) is read
// by the step, where a model has that many.
__device__ __forceinline__ void staged_load(Staged &st, uint32_t k)
{
    const unsigned char *r = smem + st.rec + k * kRecordBytes;
    st.a = *reinterpret_cast<const uint4 *>(r);
    st.b = *reinterpret_cast<const uint4 *>(r + 16);
    const double2 t = *reinterpret_cast<const double2 *>(r + 64);
    st.ts = t.x;
    st.slo = t.y;
}

// Decodes requests [i0, i0 + 32), one per lane (those past the end of the trace repeat the
// last one and are never executed).
__device__ __forceinline__ void staged_decode(Lane &ln, const Pipe &p, Staged &st, int32_t i0)
{
    const int lane = threadIdx.x & (kLanes - 1);
    __syncwarp();                                // nobody still reads the old records
    auto element = [&](int64_t first, double &ts, float &slo, int32_t &m) {
        const int64_t want = first + lane;
        const size_t o = (size_t)(want < p.last ? want : (int64_t)p.last) * p.pitch;
        ts = __ldg(p.arrivals + o);
        slo = __ldg(p.slos + o);
        m = __ldg(p.model_ids + o);
    };
    double ts;
    float slo;
    int32_t m_raw;
    if (st.ahead_base == i0) {                   // fetched while the previous block ran
        ts = st.ahead_ts; slo = st.ahead_slo; m_raw = st.ahead_m;
    } else {
        element(i0, ts, slo, m_raw);
    }
    const int64_t next0 = (int64_t)i0 + kStageAhead;
    element(next0, st.ahead_ts, st.ahead_slo, st.ahead_m);
    st.ahead_base = next0 < 0x7FFFFFFF ? (int32_t)next0 : -0x40000000;
    const int32_t m = clean_model(ln, m_raw);
    const uint4 r = fetch_row(ln, m);
    const uint4 r2 = fetch_row_b(ln, m, r);
    const uint32_t e[8] = {r.x, r.y, r.z, r.w, r2.x, r2.y, r2.z, r2.w};
    const uint32_t mrow = (uint32_t)(m < 0 ? 0 : m) * ln.C;
    uint32_t wa[8], wb[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (e[k] < kMoreReplicas) {
            const uint32_t last = rep_last(e[k]), ns = rep_stages(e[k]);
            wa[k] = (ln.clk + last * kLanes) | ((ln.clk + (last + 1 - ns) * kLanes) << 16);
            wb[k] = (ln.lat_sm + (mrow + rep_column(e[k])) * ln.S) | (ns << 16) |
                    (rep_group(e[k]) << 24);
        } else {
            wa[k] = 0xFFFFFFFFu;
            wb[k] = 0;
        }
    }
    unsigned char *rec = smem + st.rec + (uint32_t)lane * kRecordBytes;
    *reinterpret_cast<uint4 *>(rec) = make_uint4(wa[0], wa[1], wa[2], wa[3]);
    *reinterpret_cast<uint4 *>(rec + 16) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
    *reinterpret_cast<uint4 *>(rec + 32) = make_uint4(wa[4], wa[5], wa[6], wa[7]);
    *reinterpret_cast<uint4 *>(rec + 48) = make_uint4(wb[4], wb[5], wb[6], wb[7]);
    *reinterpret_cast<double2 *>(rec + 64) = make_double2(ts, (double)slo);
    st.base = i0;
    st.next = -1;
    __syncwarp();
}

// Executes request i from its record (controller.py:579-622) and returns finish - arrival.
__device__ __forceinline__ double staged_step(Lane &ln, const Pipe &p, Staged &st, int32_t i,
                                              bool record)
{
    if ((uint32_t)(i - st.base) >= (uint32_t)kStageAhead) staged_decode(ln, p, st, i);
    const uint32_t k = (uint32_t)(i - st.base);
    if (st.next != i) staged_load(st, k);
    const uint4 A = st.a, B = st.b;
    const double ts = st.ts, slo = st.slo;
    const unsigned char *second = smem + st.rec + k * kRecordBytes + 32;
    // the next request's record, before this request's stores (which the compiler could not
    // move the loads across)
    const uint32_t kn = k + 1 < (uint32_t)kStageAhead ? k + 1 : k;
    staged_load(st, kn);
    st.next = kn == k + 1 ? i + 1 : -1;

    // :589-598 replica whose last-stage clock is strictly smallest (a row is filled from
    // word 0 on)
    double best = kInf;
    uint32_t pa = 0xFFFFFFFFu, pb = 0;
    if (A.x != 0xFFFFFFFFu) {
        const double c0 = SM_F64(A.x & 0xFFFFu);
        if (c0 < best) { best = c0; pa = A.x; pb = B.x; }
        if (A.y != 0xFFFFFFFFu) {
            const double c1 = SM_F64(A.y & 0xFFFFu);
            if (c1 < best) { best = c1; pa = A.y; pb = B.y; }
            if (A.z != 0xFFFFFFFFu) {
                const double c2 = SM_F64(A.z & 0xFFFFu);
                if (c2 < best) { best = c2; pa = A.z; pb = B.z; }
                if (A.w != 0xFFFFFFFFu) {
                    const double c3 = SM_F64(A.w & 0xFFFFu);
                    if (c3 < best) { best = c3; pa = A.w; pb = B.w; }
                    const uint4 A2 = *reinterpret_cast<const uint4 *>(second);
                    const uint4 B2 = *reinterpret_cast<const uint4 *>(second + 16);
                    if (A2.x != 0xFFFFFFFFu) {               // replicas five to eight
                        const double c4 = SM_F64(A2.x & 0xFFFFu);
                        if (c4 < best) { best = c4; pa = A2.x; pb = B2.x; }
                        if (A2.y != 0xFFFFFFFFu) {
                            const double c5 = SM_F64(A2.y & 0xFFFFu);
                            if (c5 < best) { best = c5; pa = A2.y; pb = B2.y; }
                            if (A2.z != 0xFFFFFFFFu) {
                                const double c6 = SM_F64(A2.z & 0xFFFFu);
                                if (c6 < best) { best = c6; pa = A2.z; pb = B2.z; }
                                if (A2.w != 0xFFFFFFFFu) {
                                    const double c7 = SM_F64(A2.w & 0xFFFFu);
                                    if (c7 < best) { best = c7; pa = A2.w; pb = B2.w; }
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    double fin = ts;
    uint32_t rec = 0;
    if (pa != 0xFFFFFFFFu) {
        const uint32_t ck = pa >> 16, lr = pb & 0xFFFFu, ns = (pb >> 16) & 0xFFu;
        bool accept = false;
        double f = ts;
        auto run = [&](auto depth) {
            constexpr int kDepth = decltype(depth)::value;
            double c[kDepth], l[kDepth], t[kDepth];
#pragma unroll
            for (int s = 0; s < kDepth; ++s) {
                c[s] = SM_F64(ck + s * kLanes);
                l[s] = SM_F64(lr + s);
            }
            double cur = ts;
#pragma unroll
            for (int s = 0; s < kDepth; ++s) {           // :605-608
                cur = tmax(cur, c[s]) + l[s];
                t[s] = cur;
            }
            f = cur + kOverhead;                         // :610
            accept = f - ts <= slo;                      // :613
            if (accept) {
#pragma unroll
                for (int s = 0; s < kDepth; ++s) SM_F64(ck + s * kLanes) = t[s];
            }
        };
        switch (ns) {
            case 1: run(std::integral_constant<int, 1>{}); break;
            case 2: run(std::integral_constant<int, 2>{}); break;
            case 4: run(std::integral_constant<int, 4>{}); break;
            case 8: run(std::integral_constant<int, 8>{}); break;
            default: {
                double cur = ts;
                for (uint32_t s = 0; s < ns; ++s)
                    cur = tmax(cur, SM_F64(ck + s * kLanes)) + SM_F64(lr + s);
                f = cur + kOverhead;
                accept = f - ts <= slo;
                if (accept) {                             // the same chain again, stored
                    cur = ts;
                    for (uint32_t s = 0; s < ns; ++s) {
                        cur = tmax(cur, SM_F64(ck + s * kLanes)) + SM_F64(lr + s);
                        SM_F64(ck + s * kLanes) = cur;
                    }
                }
            }
        }
        if (accept) fin = f;
        rec = ((pb >> 24) + 1u) | (accept ? 0x80u : 0u);
    }
    if (record) {
        ln.dec_word |= rec << (8 * (i & 3));
        if ((i & 3) == 3 || i == p.last) {
            static_cast<uint32_t *>(ln.dec)[(size_t)(i >> 2) * ln.dec_pitch] = ln.dec_word;
            ln.dec_word = 0;
        }
    }
    return fin - ts;
}

}  // namespace mms
