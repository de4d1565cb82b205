"""The slot scheduler: admits requests into free decoder slots and evicts finished ones between graph replays.

Restates the decoder thread of the reference's Pipeline (kernels/pipeline.py:183-250) as a single-threaded driver
over any object with the StreamDecoder API:

  * free slots are a LIFO list (pipeline.py:78, 140); a request takes one when it is admitted;
  * admission happens only between steps: cross K/V are written first (fill_cross), then `admit` and a new active
    list (`set_active`) whenever the set of live slots changed (pipeline.py:199-210);
  * the host reads the end flags LAG (= 1) steps behind the newest launch, so the GPU never waits for it
    (pipeline.py:67, 217-231); a slot's flag is trusted only from a step launched after the slot was admitted
    (`admitted_at`, pipeline.py:189, 204, 222), because an older step may still be copying the previous occupant's flag;
  * eviction = drop from the active list, copy the slot's output row to pinned host memory on the decoder stream, and
    free the slot only when that copy has completed (pipeline.py:223-239);
  * the delivered tokens are out[:plen + (first eos + 1 | min(len, max_new))] (pipeline.py:241-247).

With a decoder whose active list lives on the device (`decoder.device_sched`: `admit` appends the new slots, every
step drops the rows that ended) the host never sends a row list: it only picks the bucket that holds its own count of
slots not yet evicted, which is never less than the device's live count.

Requests arrive in virtual time measured in decoding steps (`request.arrival`), so a seeded stream gives the same
schedule on every run; when nothing is live the clock jumps to the next arrival. The encoder of the reference is out
of scope here: `memory_of(request)` supplies the encoder output (frames, enc_dim) of a request, on the host or the
device.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class SchedulerStats:
    steps: int = 0
    row_steps: int = 0          # live rows summed over steps (includes prompt-feeding steps and LAG re-runs)
    padded_row_steps: int = 0   # bucket sizes summed over steps
    slot_steps: int = 0         # slots * steps, the denominator of occupancy
    steady_row_steps: int = 0   # the same two over the steady part of the stream: from the first step with 90 % of the
    steady_slot_steps: int = 0  # slots live until the last request has been admitted (no ramp-up, no drain)
    admitted: int = 0
    evicted: int = 0
    new_tokens: int = 0         # generated (non-prompt) tokens delivered
    delivered_tokens: int = 0   # prompt + generated
    idle_jumps: int = 0
    bytes: int = 0              # algorithmic HBM bytes of all steps (when the decoder reports them)
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    bucket_steps: dict = field(default_factory=dict)

    @property
    def occupancy(self) -> float:
        return self.row_steps / self.slot_steps if self.slot_steps else 0.0

    @property
    def steady_occupancy(self) -> float:
        return self.steady_row_steps / self.steady_slot_steps if self.steady_slot_steps else 0.0


class DecodeScheduler:
    LAG = 1
    CHUNK_FRAMES = 3000  # encoder frames per fill_cross call (pipeline.py:64)

    def __init__(self, decoder, memory_of, *, account_bytes: bool = False, trace: list | None = None):
        self.dec = decoder
        self.memory_of = memory_of
        self.cuda = isinstance(getattr(decoder, "out", None), torch.Tensor) and decoder.out.is_cuda
        self.free = list(range(decoder.slots))[::-1]
        self.account_bytes = account_bytes
        self.trace = trace
        self.stats = SchedulerStats()
        self.device_sched = bool(getattr(decoder, "device_sched", False))
        self.step_ms: deque = deque(maxlen=4096)  # device time between the ends of consecutive steps, newest last
        self._prev_ev = None
        cols = decoder.out.shape[1]
        if self.cuda:
            self.out_host = torch.zeros(decoder.slots + 1, cols, dtype=torch.long).pin_memory()
            self.fill_stream = torch.cuda.Stream(device=decoder.device)
        else:
            self.out_host = np.zeros((decoder.slots + 1, cols), np.int64)

    # ---- backend shims (CUDA decoder or the CPU oracle with the same API) ------------------------------------------

    def _event(self):
        if not self.cuda:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(self.dec.stream)
        return ev

    def step_time_summary(self) -> dict:
        """p50 / p90 / p99 / max of the recorded step times in ms (the reference keeps per-stage times in
        Pipeline.stats, kernels/pipeline.py:82-83, 172-178)."""
        if not self.step_ms:
            return {}
        v = np.sort(np.asarray(self.step_ms))
        pick = lambda q: float(v[min(len(v) - 1, int(q * len(v)))])  # noqa: E731
        return {"steps": len(v), "p50_ms": pick(0.5), "p90_ms": pick(0.9), "p99_ms": pick(0.99), "max_ms": float(v[-1])}

    def _flags(self) -> np.ndarray:
        f = self.dec.flags
        return f.numpy() if isinstance(f, torch.Tensor) else f

    def _fill(self, reqs, slots) -> None:
        lengths = [r.frames for r in reqs]
        mems = [self.memory_of(r) for r in reqs]
        if not self.cuda:
            self.dec.fill_cross(np.concatenate([np.asarray(m) for m in mems]), lengths, slots)
            return
        with torch.cuda.stream(self.fill_stream):
            parts = []
            for m in mems:
                m = torch.as_tensor(m)
                if not m.is_cuda:
                    self.stats.h2d_bytes += m.numel() * m.element_size()
                    m = m.to(self.dec.device, non_blocking=True)
                parts.append(m)
            self.dec.fill_cross(torch.cat(parts), lengths, slots)
            done = torch.cuda.Event()
            done.record(self.fill_stream)
        self.dec.stream.wait_event(done)  # the decoder stream's next work is ordered after the cache writes

    def _copy_out(self, slot: int):
        if self.cuda:
            self.out_host[slot].copy_(self.dec.out[slot], non_blocking=True)
            self.stats.d2h_bytes += self.dec.out.shape[1] * 8
        else:
            self.out_host[slot] = self.dec.out[slot]

    # ---- the loop ----------------------------------------------------------------------------------------------------

    def _deliver(self, req, row: np.ndarray) -> np.ndarray:
        plen = len(req.prompt)
        gen = row[plen:]
        end = np.nonzero(gen == self.dec.eos)[0]
        max_new = min(getattr(req, "target", self.dec.max_new_tokens), self.dec.max_new_tokens)
        n = plen + (end[0] + 1 if len(end) else min(len(gen), max_new))
        self.stats.new_tokens += n - plen
        self.stats.delivered_tokens += n
        return row[:n].copy()

    def run(self, requests, max_steps: int | None = None, on_step=None) -> list:
        """Decode every request of the stream; returns the token arrays (prompt + generated) in request order.
        on_step(step_no, bucket, active slots) is called after each launch (used by the benchmark to time steps)."""
        dec, st = self.dec, self.stats
        waiting = deque(sorted(range(len(requests)), key=lambda i: requests[i].arrival))
        results: list = [None] * len(requests)
        active: list[int] = []
        req_of: dict[int, int] = {}
        admitted_at: dict[int, int] = {}
        steps: deque = deque()
        copies: deque = deque()
        pos_of: dict[int, int] = {}  # host mirror of each live slot's position, for byte accounting
        step_no, clock, bucket, changed, ramped = 0, 0.0, 1, False, False
        while waiting or active or copies or steps:
            # -- admit what has arrived and fits
            new_slots, new_idx, frames = [], [], 0
            while waiting and self.free and requests[waiting[0]].arrival <= clock:
                r = requests[waiting[0]]
                if new_idx and frames + r.frames > self.CHUNK_FRAMES:
                    break
                new_idx.append(waiting.popleft())
                new_slots.append(self.free.pop())
                frames += r.frames
            if new_idx:
                new_reqs = [requests[i] for i in new_idx]
                self._fill(new_reqs, new_slots)
                dec.admit(new_slots, [torch.as_tensor(r.prompt) if self.cuda else r.prompt for r in new_reqs],
                          [r.frames for r in new_reqs],
                          [min(getattr(r, "target", dec.max_new_tokens), dec.max_new_tokens) for r in new_reqs])
                for s, i in zip(new_slots, new_idx):
                    req_of[s], admitted_at[s], pos_of[s] = i, step_no, 0
                active += new_slots
                st.admitted += len(new_slots)
                changed = True
                if self.trace is not None:
                    self.trace.append((step_no, "admit", list(new_slots)))
            # -- one step over the live slots
            if active:
                if changed:
                    bucket = dec.bucket(len(active)) if self.device_sched else dec.set_active(active)
                    changed = False
                if self.account_bytes:
                    st.bytes += dec.step_bytes([pos_of[s] for s in active],
                                               [requests[req_of[s]].frames for s in active], bucket)
                dec.step(bucket)
                steps.append((step_no, self._event()))
                if on_step is not None:
                    on_step(step_no, bucket, active)
                for s in active:
                    r = requests[req_of[s]]
                    pos_of[s] = min(pos_of[s] + 1, len(r.prompt) - 1 + min(r.target, dec.max_new_tokens))
                st.steps += 1
                st.row_steps += len(active)
                st.padded_row_steps += bucket
                st.slot_steps += dec.slots
                ramped = ramped or len(active) >= 0.9 * dec.slots
                if ramped and waiting:
                    st.steady_row_steps += len(active)
                    st.steady_slot_steps += dec.slots
                st.bucket_steps[bucket] = st.bucket_steps.get(bucket, 0) + 1
                step_no += 1
                clock = max(clock, float(step_no))
            elif waiting and not copies and not steps:
                clock = max(clock, requests[waiting[0]].arrival)  # idle: jump to the next arrival
                st.idle_jumps += 1
            # -- end flags of the step LAG behind the newest (of every step when nothing runs)
            while steps and (len(steps) > self.LAG or not active):
                k, ev = steps.popleft()
                if ev is not None:
                    ev.synchronize()
                    if self._prev_ev is not None and self._prev_ev[0] == k - 1:
                        self.step_ms.append(self._prev_ev[1].elapsed_time(ev))
                    self._prev_ev = (k, ev)
                flags = self._flags()
                ended = [s for s in active if flags[s] and admitted_at[s] <= k]
                if ended:
                    gone = set(ended)
                    active = [s for s in active if s not in gone]
                    changed = True
                    if self.cuda:
                        torch.cuda.nvtx.range_push("b200dec.evict")
                        with torch.cuda.stream(dec.stream):
                            for s in ended:
                                self._copy_out(s)
                            cev = self._event()
                        torch.cuda.nvtx.range_pop()
                    else:
                        for s in ended:
                            self._copy_out(s)
                        cev = None
                    copies.append((cev, [(s, req_of.pop(s)) for s in ended]))
                    if self.trace is not None:
                        self.trace.append((step_no, "evict", list(ended)))
            # -- completed copies: deliver, free the slots
            while copies and (copies[0][0] is None or copies[0][0].query() or not active):
                cev, rows = copies.popleft()
                if cev is not None:
                    cev.synchronize()
                for s, i in rows:
                    row = self.out_host[s].numpy() if self.cuda else self.out_host[s]
                    results[i] = self._deliver(requests[i], row)
                    self.free.append(s)
                    pos_of.pop(s, None)
                    st.evicted += 1
            if max_steps is not None and step_no >= max_steps:
                break
        return results
