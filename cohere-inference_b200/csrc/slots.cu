// Slot bookkeeping on the device: admission of new requests and the active list.
//
// The host side of the reference (kernels/stream_decoder.py:241-272) writes a dozen small tensors per admission with
// indexed assignments and copies the active list on every change. Here the host stages one packed record per new
// request in pinned memory, one asynchronous copy brings the batch over, and one kernel writes every slot field; the
// same kernel can append the slots to the device's own active list, and a small kernel at the tail of a step drops
// the rows that ended from that list, so the list never has to travel (the slot scheduler then only watches the end
// flags and the live count the step leaves in pinned memory).
#include "common.cuh"

using namespace b200dec_detail;

namespace {

constexpr int REC_HEAD = 4;  // slot, prompt length, new-token budget, encoder frames; then max_prompt token ids

struct AdmitArgs {
  const int32_t* rec;
  int n, slots, max_prompt, out_cols, pad, frames, max_rows;
  int64_t* tok;
  int32_t* pos;
  int32_t* plen;
  int32_t* limit;
  int32_t* cross_len;
  uint8_t* finished;
  int64_t* forced;
  int64_t* out;
  int32_t* active;    // with n_active: the list the slots are appended to
  int32_t* n_active;  // or null
  int32_t* status;
};

// One CTA, the requests one after another (at most a few hundred, a few microseconds): the appends keep their order.
__global__ void __launch_bounds__(128) admit_kernel(const AdmitArgs p) {
  const int tid = threadIdx.x, stride = REC_HEAD + p.max_prompt;
  const int base = p.n_active ? *p.n_active : 0;
  int appended = 0;
  for (int i = 0; i < p.n; ++i) {
    const int32_t* r = p.rec + (size_t)i * stride;
    const int s = r[0];
    int plen = r[1], frames = r[3];
    const int budget = r[2];
    if (s < 0 || s >= p.slots) {  // uniform across the CTA: skip the record
      if (tid == 0) atomicOr(p.status, B200DEC_ST_SLOT_RANGE);
      continue;
    }
    if (plen < 1 || plen > p.max_prompt) {
      if (tid == 0) atomicOr(p.status, B200DEC_ST_POS_RANGE);
      plen = plen < 1 ? 1 : p.max_prompt;
    }
    if (frames < 1 || frames > p.frames) {
      if (tid == 0) atomicOr(p.status, B200DEC_ST_FRAMES_RANGE);
      frames = frames < 1 ? 1 : p.frames;
    }
    for (int c = tid; c < p.max_prompt; c += blockDim.x)
      p.forced[(size_t)s * p.max_prompt + c] = c < plen ? (int64_t)r[REC_HEAD + c] : (int64_t)p.pad;
    for (int c = tid; c < p.out_cols; c += blockDim.x)
      p.out[(size_t)s * p.out_cols + c] = c < plen ? (int64_t)r[REC_HEAD + c] : (int64_t)p.pad;
    if (tid == 0) {
      p.tok[s] = r[REC_HEAD];
      p.pos[s] = 0;
      p.plen[s] = plen;
      p.limit[s] = plen - 1 + budget;
      p.cross_len[s] = frames;
      p.finished[s] = 0;
      if (p.n_active) {
        if (base + appended < p.max_rows) p.active[base + appended] = s;
        else atomicOr(p.status, B200DEC_ST_SLOT_RANGE);
      }
    }
    ++appended;
  }
  if (p.n_active && tid == 0) *p.n_active = min(base + appended, p.max_rows);
}

struct CompactArgs {
  int32_t* active;
  int32_t* n_active;
  int32_t* live_host;  // pinned host memory mapped into the device's address space, or null: the live count
  const uint8_t* finished;
  int rows, dummy;
};

// The live rows of active[0 .. rows) to the front in their order, the rest on the dummy slot; one thread per row.
__global__ void __launch_bounds__(128) compact_kernel(const CompactArgs p) {
  __shared__ int s_warp[4];
  const int r = threadIdx.x, lane = r & 31, warp = r >> 5;
  pdl_wait();
  pdl_trigger();
  const int n = *p.n_active;
  int s = p.dummy;
  bool live = false;
  if (r < p.rows && r < n) {
    s = p.active[r];
    live = s >= 0 && s < p.dummy && !p.finished[s];
  }
  const unsigned m = __ballot_sync(0xffffffffu, live);
  if (lane == 0) s_warp[warp] = __popc(m);
  __syncthreads();
  int before = __popc(m & ((1u << lane) - 1));
  int total = 0;
  for (int w = 0; w < 4; ++w) {
    if (w < warp) before += s_warp[w];
    total += s_warp[w];
  }
  __syncthreads();  // every row has been read
  if (live) p.active[before] = s;
  if (r >= total && r < p.rows) p.active[r] = p.dummy;
  if (r == 0) {
    *p.n_active = total;
    if (p.live_host) *p.live_host = total;
  }
}

}  // namespace

extern "C" {

int b200dec_admit_record_ints(int max_prompt) { return REC_HEAD + max_prompt; }

int b200dec_admit(const b200dec_plan* pl, const int32_t* records, int n, int32_t* n_active, int max_rows, void* stream) {
  B200_REQUIRE(pl && records && pl->tok && pl->pos && pl->plen && pl->limit && pl->cross_len && pl->finished &&
                   pl->forced && pl->out && pl->status, "admit: null pointer");
  B200_REQUIRE(n >= 0 && pl->max_prompt >= 1 && pl->out_cols >= pl->max_prompt, "admit: n %d max_prompt %d out_cols %d", n,
               pl->max_prompt, pl->out_cols);
  B200_REQUIRE(!n_active || (pl->active && max_rows >= 1), "admit: appending needs the active list and its capacity");
  if (n == 0) return 0;
  AdmitArgs a{records, n, pl->slots, pl->max_prompt, pl->out_cols, pl->pad, pl->frames, max_rows, pl->tok, pl->pos,
              const_cast<int32_t*>(pl->plen), const_cast<int32_t*>(pl->limit), const_cast<int32_t*>(pl->cross_len),
              pl->finished, const_cast<int64_t*>(pl->forced), pl->out, const_cast<int32_t*>(pl->active), n_active,
              pl->status};
  admit_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(a);
  return check_launch("admit");
}

int b200dec_compact_active(const b200dec_plan* pl, int rows, int32_t* n_active, int32_t* live_host, int pdl,
                           void* stream) {
  B200_REQUIRE(pl && pl->active && pl->finished && n_active, "compact_active: null pointer");
  B200_REQUIRE(rows >= 1 && rows <= 128, "compact_active: rows %d (1..128)", rows);
  CompactArgs a{const_cast<int32_t*>(pl->active), n_active, live_host, pl->finished, rows, pl->slots};
  const cudaError_t e = launch_kernel(compact_kernel, dim3(1), dim3(128), 0, (cudaStream_t)stream, 0, pdl != 0, a);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "compact_active launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
