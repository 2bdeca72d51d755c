"""Streaming ("live") load on one model: every participant owns a ring of device token slots, each hop uploads its new
crops and scores the window of its last 20 frames.

Host-side mirror of the reference's live benchmark driver (bench/gpu_bench.cpp:141-218): participant p owns token slots
[p*24, p*24 + 24); frame number k of p lives in slot p*24 + k % 24; a hop is one request per participant that carries
`new` crops (`frames`), stores their tokens into the ring (`store_slots`) and builds one window from the 20 most recent
ring slots (`window_slots`).  The first hop of a participant carries 20 crops.  Across the GPUs of a box a participant
stays on one device (`sharding.device_of_participant`), so its ring never moves.
"""
from __future__ import annotations

import numpy as np

RING = 24
WINDOW = 20


def ring_slot(participant: int, frame_number: int) -> int:
    """Device token slot that holds frame `frame_number` (0, 1, 2, ...) of `participant`."""
    if participant < 0 or frame_number < 0:
        raise ValueError("negative participant or frame number")
    return participant * RING + frame_number % RING


def hop_slots(participant: int, frames_so_far: int, new: int):
    """(store_slots [new], window_slots [20]) of the hop that appends `new` crops to a participant that has already
    sent `frames_so_far`: the window covers frames [frames_so_far + new - 20, frames_so_far + new)."""
    if new < 1 or new > RING - 1:
        raise ValueError("a hop carries 1 .. 23 crops")
    last = frames_so_far + new
    if last < WINDOW:
        raise ValueError("the first hop of a participant must bring the window to 20 frames")
    store = np.array([ring_slot(participant, frames_so_far + i) for i in range(new)], np.int32)
    window = np.array([ring_slot(participant, last - WINDOW + s) for s in range(WINDOW)], np.int32)
    return store, window


def place_participants(participant_ids, world: int):
    """Per device of a box: the positions (in `participant_ids`) of the participants whose rings live there, in input
    order; a participant's local ring index on its device is its position in that list.  Placement is the stable hash
    of sharding.device_of_participant, so a participant keeps its device (and its 24 token slots) for the whole call."""
    from .sharding import device_of_participant

    placed = [[] for _ in range(world)]
    for i, pid in enumerate(participant_ids):
        placed[device_of_participant(pid, world)].append(i)
    return placed


class LiveDriver:
    """Drives hops of `participants` rings through one binding.CudaModel (which must have token_slots >= 24 * participants)."""

    def __init__(self, model, participants: int):
        limits = model.limits()
        if limits["token_slots"] < RING * participants:
            raise ValueError(f"model has {limits['token_slots']} token slots, {RING * participants} needed")
        self.model = model
        self.participants = participants
        self.frames_sent = np.zeros(participants, np.int64)

    def hop(self, crops):
        """crops: uint8 [participants, new, 180, 320, 3] (the same `new` for all).  Submits one request per participant,
        waits for all of them and returns (logits [participants], timings: list of shv_cuda_job_timing dicts)."""
        crops = np.ascontiguousarray(crops, dtype=np.uint8)
        if crops.ndim != 5 or crops.shape[0] != self.participants or crops.shape[2:] != (180, 320, 3):
            raise ValueError("expected uint8 crops [participants, new, 180, 320, 3]")
        new = crops.shape[1]
        logits = np.full(self.participants, np.nan, np.float32)
        jobs, keep = [], []
        for p in range(self.participants):
            store, window = hop_slots(p, int(self.frames_sent[p]), new)
            job, k = self.model.submit(1, logits[p:p + 1], window_slots=window, frames=crops[p], n_frames=new, store_slots=store)
            if not job:
                from . import binding
                err = binding.last_error(self.model.L)
                for j in jobs:
                    self.model.job_wait(j)
                    self.model.job_free(j)
                raise RuntimeError(err)
            jobs.append(job)
            keep.append(k)
            self.frames_sent[p] += new
        timings, failed = [], None
        for j in jobs:
            if self.model.job_wait(j) != 0 and failed is None:
                failed = self.model.job_error(j)
            timings.append(self.model.job_timing(j)[1])
            self.model.job_free(j)
        if failed:
            raise RuntimeError(failed)
        return logits, timings


class BoxLiveDriver:
    """The same hops over the GPUs of a box behind one binding.Box: a participant's session is opened on its home
    device (crc32 of its id modulo the number of devices, spilling when that device is full), its ring is the block of 24
    token slots the box handed out there, and every hop request of the participant goes to that device."""

    def __init__(self, box, participant_ids):
        self.box = box
        self.ids = list(participant_ids)
        self.sessions = [box.session_open(pid) for pid in self.ids]            # (device, first slot of the ring)
        self.frames_sent = np.zeros(len(self.ids), np.int64)

    def ring_slots(self, p: int, new: int):
        """(store_slots, window_slots) of participant p's next hop, in the slot numbering of its device."""
        store, window = hop_slots(0, int(self.frames_sent[p]), new)
        base = self.sessions[p][1]
        return store + base, window + base

    def hop(self, crops_of, new: int):
        """crops_of(p) -> uint8 array [new, 180, 320, 3] (pinned memory is DMA'd without staging).  One request per
        participant to its device; returns (logits [participants], batch sizes seen by the jobs)."""
        from . import binding
        L = self.box.L
        n = len(self.ids)
        logits = np.full(n, np.nan, np.float32)
        jobs, keep = [], []
        for p in range(n):
            store, window = self.ring_slots(p, new)
            req, k = binding.build_request(1, logits[p:p + 1], window_slots=window, frames=crops_of(p), n_frames=new, store_slots=store)
            job = self.box.submit(self.sessions[p][0], req)
            if not job:
                err = binding.last_error(L)
                for j in jobs:
                    L.shv_cuda_job_wait(j)
                    L.shv_cuda_job_free(j)
                raise RuntimeError(err)
            jobs.append(job)
            keep.append(k)
            self.frames_sent[p] += new
        sizes, failed = [], None
        bw = binding.C.c_int()
        for j in jobs:
            if L.shv_cuda_job_wait(j) != 0 and failed is None:
                failed = L.shv_cuda_job_error(j).decode()
            L.shv_cuda_job_timing(j, None, None, None, None, binding.C.byref(bw))
            sizes.append(bw.value)
            L.shv_cuda_job_free(j)
        if failed:
            raise RuntimeError(failed)
        return logits, sizes
