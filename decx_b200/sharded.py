"""Row-sharded GEMM over the GPUs of one box, one process per GPU (torch.distributed).

    D (M x N, on the owner)  =  A (M x K, rows partitioned over the ranks)  .  B (K x N, on the owner)

The reference is single-GPU (its sources hold no cudaSetDevice, peer copy or collective), so this
layer is new surface on top of the same per-GPU GEMM.  One step is:

  1. B travels from the owner to every rank in column panels on a communication stream: the owner packs
     panel j into a contiguous K x Np buffer; then either one NCCL broadcast ("broadcast"), or -- the
     default for more than two ranks, because an 8-rank ncclBroadcast only reaches ~150 GB/s here -- the
     owner scatters one row block of the panel to each rank and an all-gather completes it everywhere
     ("scatter_allgather": every link of the NVSwitch fabric carries a share, the owner sends the panel once);
     or "p2p": the same scatter + all-gather pattern done by the copy engines -- the panel buffers live in
     symmetric memory, every rank PULLS its row block from the owner and then the other blocks from the
     ranks that hold them, ordered by stream-level signals, so no communication kernel competes with the
     persistent GEMM for SMs;
  2. as soon as panel j has landed in this rank's own HBM, the rank's GEMM for that panel runs on the
     compute stream, D[rows of this rank, panel j] = A_r . B[:, panel j]  (its TMA loads read local
     memory only, none of them uses cluster multicast), while panel j+1 is still in flight;
  3. gather on the owner, mode "peer" (default on GPUs): the owner's D is exported through a CUDA IPC
     handle and each rank's GEMM epilogue stores its rows straight into it over NVLink, so the
     gather is fused into the kernel and finished when the kernels are; mode "collective": each rank
     keeps a local D shard and sends it to the owner afterwards (plain point-to-point; this is the
     form the CPU tests run over gloo with an injected host GEMM);
  4. a barrier across the ranks closes the step.

fp16 on GPUs runs steps 1 and 2 as ONE kernel launch per rank ("single" overlap): every rank keeps a full
row-major replica of B in symmetric memory, the copy engines fill it panel by panel (same pull pattern as
"p2p", 2-D copies) and write a flag per panel with a stream memory operation; the GEMM is launched at once,
walks its tiles panel by panel and its loader waits on a panel's flag before touching it
(decxb200_gemm_fp16_panels).  No per-panel launches, so no round of the persistent grid is left half empty
at a panel boundary, and the 256 x 512 tile applies.

"fused" overlap (the default for fp16 on GPUs) goes one step further and needs no copy engine, no communication
stream and no NCCL call inside the step: the GEMM kernel itself brings B in (decxb200_gemm_fp16_fetch).  Every
CTA carries two courier warps, and its epilogue warps join in while their tile is being multiplied.  The OWNER's
couriers push one row piece of each panel into every other rank's replica and raise that rank's publish flag
(scatter: the owner sends every byte once, with posted stores); the other ranks' couriers wait for their own
piece and copy the remaining pieces from the ranks that hold them (all-gather), panel by panel, with 16-byte
peer loads.  The tiles of a panel
start when its pieces are counted complete.  One launch per rank does broadcast, product and -- through D in
the owner's memory -- the gather; two stream-ordered symmetric-memory barriers bracket it.

Rows are dealt in multiples of 256 (the CTA-pair tile height), so every rank runs whole tiles.
"""
import ctypes

import torch
import torch.distributed as dist

ROW_ALIGN = 256
COL_ALIGN = 256


def row_ranges(M, world, align=ROW_ALIGN, lighter=None):
    """[(first_row, rows)] per rank: equal blocks of whole `align`-row tiles, the remainder on the
    last ranks that still get rows; ranks beyond the data get (M, 0).

    lighter = (rank, k): that rank gets k blocks fewer and the others share them (the owner of B spends part of
    its SMs' time sending B; with a smaller share it finishes together with the others).  Ignored when the
    matrix has too few blocks for it."""
    blocks = (M + align - 1) // align
    per = (blocks + world - 1) // world
    counts = [max(0, min(per, blocks - r * per)) for r in range(world)]
    if lighter is not None and world > 1:
        rank, k = lighter
        if 0 < k < counts[rank] and all(c > 0 for c in counts):
            counts[rank] -= k
            others = [r for r in range(world) if r != rank]
            for i in range(k):
                counts[others[-1 - (i % len(others))]] += 1
    out, start = [], 0
    for r in range(world):
        first = min(M, start * align)
        stop = min(M, (start + counts[r]) * align)
        out.append((first, stop - first))
        start += counts[r]
    return out


def panel_plan(N, panels, align=COL_ALIGN):
    """[(first_col, cols)] of the column panels of B.

    `panels` is a count (near-equal multiples of `align`), a list of widths, or "ramp": a small first panel
    (N/16) so that the first tiles can start early, then 3N/16, then quarters -- nothing hides the arrival of
    the first panel, everything after it travels while tiles are being computed.  (Measured at 8 GPUs on
    65536 x 16384 x 16384: ramp 4.08-4.17 ms per step; small first AND last panel 4.30 ms.)"""
    if panels == "ramp":
        units = (N + align - 1) // align
        if units < 16:
            return panel_plan(N, min(4, units), align)
        first, second = max(1, units // 16), max(1, 3 * units // 16)
        q, extra = divmod(units - first - second, 3)
        widths = [first, second] + [q + (1 if i < extra else 0) for i in range(3)]
        panels = [w * align for w in widths if w > 0]
    if isinstance(panels, (list, tuple)):
        out, c = [], 0
        for w in panels:
            w = min(int(w), N - c)
            if w > 0:
                out.append((c, w))
                c += w
        if c < N:
            out.append((c, N - c))
        return out
    blocks = (N + align - 1) // align
    panels = max(1, min(panels, blocks))
    base, extra = divmod(blocks, panels)
    out, c = [], 0
    for j in range(panels):
        w = (base + (1 if j < extra else 0)) * align
        w = min(w, N - c)
        out.append((c, w))
        c += w
    assert c == N
    return out


def fetch_panel_plan(N, tile=512, max_panels=16):
    """Column panels for the fused kernel: narrow ones first (two tiles = 1024 columns) so that the first
    tiles start after a few dozen microseconds of transfer, four-tile panels afterwards (wider panels keep
    the tiles that run together on fewer rows of A)."""
    tiles = (N + tile - 1) // tile
    widths, left = [], tiles
    while left > 0:
        w = 2 if len(widths) < 4 else 4
        w = min(w, left)
        widths.append(w)
        left -= w
    while len(widths) > max_panels:                 # very wide B: merge the last panels pairwise
        widths[-2:] = [widths[-2] + widths[-1]]
    return panel_plan(N, [w * tile for w in widths])


def row_pieces(K, parts, align=16):
    """[(first_row, rows)]: K rows of B cut into `parts` near-equal pieces (multiples of `align` rows)."""
    units = (K + align - 1) // align
    base, extra = divmod(units, parts)
    out, r = [], 0
    for i in range(parts):
        n = min((base + (1 if i < extra else 0)) * align, K - r)
        out.append((r, n))
        r += n
    return out


def fetch_jobs(rank, owner, active, K, panels, b_ptr, pub_ptr, scatter="push", mc_ptr=None, mc_pub_ptr=None):
    """Job list of `rank` for the fused kernel, as tuples
    (src, gate, row0, rows, col0, cols, panel, publish, dst, notify).

    `active` are the ranks that run a kernel (they have rows of A).  The non-owners among them ("holders") each
    become the first holder of one row piece of every panel and fetch the remaining pieces from each other, gated
    on the holder's publish flag for the panel.  How a holder gets its own piece:
      scatter="push" (default): the OWNER's couriers store it into the holder's replica and then set the holder's
          publish flag (posted stores: no request travels towards the owner, whose inbound link carries D); the
          holder lists the piece as a rows == 0 job gated on its own flag;
      scatter="pull": the holder's couriers read it from the owner's B and publish it themselves.
      scatter="multicast": no pieces at all.  The owner's couriers store every panel ONCE through the NVLink
          multicast mapping of the replicas (mc_ptr) and raise everybody's publish flag through the multicast
          mapping of the flags (mc_pub_ptr); every other rank lists one rows == 0 job per panel gated on its own flag.
    b_ptr[r] / pub_ptr[r]: address of rank r's replica of B / of its publish flags, as this rank maps them."""
    holders = [r for r in active if r != owner]
    if rank not in active or not holders:
        return []
    if scatter == "multicast":
        if not mc_ptr or not mc_pub_ptr:
            raise ValueError("multicast scatter needs the multicast addresses of the replica and of the flags")
        if rank == owner:
            return [(b_ptr[owner], None, 0, K, c0, w, p, 2, mc_ptr, mc_pub_ptr + 4 * p) for p, (c0, w) in enumerate(panels)]
        return [(None, pub_ptr[rank] + 4 * p, 0, 0, c0, w, p, 0, None, None) for p, (c0, w) in enumerate(panels)]
    pieces = row_pieces(K, len(holders))
    jobs = []
    if rank == owner:
        if scatter != "push":
            return []
        for p, (c0, w) in enumerate(panels):
            for k in range(len(holders)):
                i = (p + k) % len(holders)                    # start every panel at another target
                r0, nr = pieces[i]
                if nr:
                    q = holders[i]
                    jobs.append((b_ptr[owner], None, r0, nr, c0, w, p, 0, b_ptr[q], pub_ptr[q] + 4 * p))
        return jobs
    me = holders.index(rank)
    for p, (c0, w) in enumerate(panels):
        r0, nr = pieces[me]
        if nr:
            if scatter == "push":
                jobs.append((None, pub_ptr[rank] + 4 * p, r0, 0, c0, w, p, 0, None, None))
            else:
                jobs.append((b_ptr[owner], None, r0, nr, c0, w, p, 1 if len(holders) > 1 else 0, None, None))
        for d in range(1, len(holders)):
            h = (me + d) % len(holders)                       # stagger the sources over the ranks
            r0, nr = pieces[h]
            if nr:
                jobs.append((b_ptr[holders[h]], pub_ptr[holders[h]] + 4 * p, r0, nr, c0, w, p, 0, None, None))
    return jobs


class _RawCuda:
    """Lets torch view memory that was allocated through the C ABI (``__cuda_array_interface__``)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 2}


_TYPESTR = {torch.float16: "<f2", torch.float32: "<f4", torch.complex64: "<c8"}


class ShardedGemm:
    """Buffers and schedule of one sharded problem; ``step()`` runs it once.

    After construction fill ``self.A`` (this rank's rows of A) and, on the owner, ``self.B``.
    The owner reads the result from ``self.D`` (M x N).  ``gemm_fn(A, Bp, out)`` replaces the CUDA
    GEMM in CPU tests only; on a GPU the C ABI is called and there is no other path.
    """

    def __init__(self, M, N, K, dtype, group=None, owner=0, panels="ramp", gather=None, device=None, gemm_fn=None,
                 reserve_sms=None, bcast=None, overlap=None, tile=0, scatter="push", owner_blocks_less=None, forward_d=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.owner, self.M, self.N, self.K, self.dtype = owner, M, N, K, dtype
        self.device = torch.device(device if device is not None else "cpu")
        self.on_gpu = self.device.type == "cuda"
        if not self.on_gpu and gemm_fn is None:
            raise RuntimeError("ShardedGemm computes on CUDA devices only (a host GEMM can only be injected by tests)")
        self.gemm_fn = gemm_fn
        self._scatter = scatter
        # D through the couriers (see the C header): measured in same-box runs +1 % at 2 GPUs (13.79 vs 13.94 ms),
        # -1.3 % at 4 (7.35 vs 7.25 ms), +0.4 % at 8 (4.14 vs 4.16 ms): on by default at 2 GPUs only
        self._forward_d = forward_d
        self.bcast = bcast or ("p2p" if self.on_gpu else "broadcast")
        # SMs left free for the communication kernels while a GEMM runs: the GEMM is persistent (one CTA per
        # SM for its whole duration), so without this NCCL's broadcast of the next panel cannot get an SM
        # until the GEMM ends and the pipeline becomes broadcast-bound.
        self._reserve_arg = reserve_sms
        self.gather = gather or ("peer" if self.on_gpu and self.world > 1 else "collective")
        if owner_blocks_less is None:
            # the owner of B also sends B and receives everybody's D: at 8 GPUs it finishes with the others when it
            # has two 256-row blocks fewer (4.04 vs 4.10, 4.07 vs 4.15, 3.98 vs 4.02 ms per step in three runs)
            owner_blocks_less = 2 if (self.world >= 8 and overlap in (None, "fused")) else 0
        self.rows = row_ranges(M, self.world, lighter=(owner, owner_blocks_less) if owner_blocks_less else None)
        self.row0, self.nrows = self.rows[self.rank]
        self.panels = panel_plan(N, panels if self.world > 1 else 1)
        self.is_owner = self.rank == owner
        dev = self.device
        self.A = torch.empty((max(self.nrows, 1), K), dtype=dtype, device=dev)[: self.nrows]
        self.B = torch.empty((K, N), dtype=dtype, device=dev) if self.is_owner else None
        self._epoch = 0
        self._hdl = None
        self.overlap = "panels"                 # one GEMM launch per panel
        if self.world > 1 and self.bcast == "p2p" and (not self.on_gpu or K % self.world != 0):
            self.bcast = "broadcast"
        if (overlap in (None, "fused") and self.world > 1 and self.on_gpu and dtype == torch.float16
                and gemm_fn is None and self.gather == "peer" and N % 8 == 0 and bcast in (None, "p2p")):
            self.panels = fetch_panel_plan(N) if panels == "ramp" else panel_plan(N, panels, align=512)
            if len(self.panels) <= 16 and self._setup_fused():
                self.overlap = "fused"
                self.bcast = "in-kernel"
        if (self.overlap != "fused" and overlap in (None, "single") and self.world > 1 and self.bcast == "p2p"
                and dtype == torch.float16 and gemm_fn is None and self.gather == "peer" and N % 8 == 0):
            self.panels = panel_plan(N, panels, align=512)
            if len(self.panels) <= 8 and self._setup_symmetric_replica():
                self.overlap = "single"
        if self.world > 1 and self.bcast == "p2p" and self.overlap not in ("single", "fused"):
            self._setup_symmetric_panels()
        if self.overlap in ("single", "fused"):
            self.Bp = None
        elif self.world > 1 and self._hdl is None:
            self.Bp = [torch.empty((K, w), dtype=dtype, device=dev) for _, w in self.panels]
        elif self.world == 1:
            self.Bp = [self.B]
        self.launches = 0
        self._peer_base = None
        self._owned = None
        esz = torch.empty(0, dtype=dtype).element_size()
        self._esz = esz
        if self.on_gpu:
            from . import capi, gemm as G
            self._capi, self._G = capi, G
            self._dt = G._DTYPES[dtype]
            self.status = G.new_status(dev)
            need = max((capi.workspace_bytes(self._dt, max(self.nrows, 1), w, K) for _, w in self.panels), default=0)
            self.workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
            self._ws_bytes = need
            # "p2p" moves B with the copy engines (its signal kernels are one tiny CTA): nothing to reserve;
            # NCCL broadcasts need SMs of their own or the pipeline becomes broadcast-bound
            self.reserve_sms = self._reserve_arg if self._reserve_arg is not None else \
                (0 if (self.world == 1 or self.bcast == "p2p") else 16)
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            self._max_ctas = max(2, sms - self.reserve_sms) if self.reserve_sms else 0
            self.comm_stream = torch.cuda.Stream(device=dev)
            self.events = [torch.cuda.Event() for _ in self.panels]
            self._tile = tile
            self.kernel_variant = 0
            if self.overlap == "fused":
                self._fused_prepare()
        if self.gather == "peer":
            self._setup_peer_d()
        else:
            self.D = torch.empty((M, N), dtype=dtype, device=dev) if self.is_owner else None
            self.D_local = self.D[self.row0:self.row0 + self.nrows] if self.is_owner else \
                torch.empty((max(self.nrows, 1), N), dtype=dtype, device=dev)[: self.nrows]

    # ------------------------------------------------------------------ B panels in symmetric memory ("p2p")
    def _setup_symmetric_panels(self):
        """All panels of B in one symmetric allocation; every rank can address every other rank's copy."""
        import sys
        try:
            import torch.distributed._symmetric_memory as symm
            total = self.K * self.N
            self._bsym = symm.empty(total, dtype=self.dtype, device=self.device)
            grp = self.group if self.group is not None else dist.group.WORLD
            self._hdl = symm.rendezvous(self._bsym, group=grp)
            self._poff, off = [], 0
            for _, w in self.panels:
                self._poff.append(off)
                off += self.K * w
            self.Bp = [self._bsym[o:o + self.K * w].view(self.K, w) for o, (_, w) in zip(self._poff, self.panels)]
            self._peer = [self._hdl.get_buffer(r, (total,), self.dtype, 0) for r in range(self.world)]
        except Exception as e:       # symmetric memory not available on this system: NCCL broadcast instead
            print(f"decx_b200.sharded: symmetric memory unavailable ({type(e).__name__}: {e}); using ncclBroadcast",
                  file=sys.stderr)
            self._hdl = None
            self.bcast = "broadcast"

    def _setup_symmetric_replica(self):
        """"single" overlap: a full K x N replica of B per rank in symmetric memory (the owner's is B itself)."""
        import sys
        try:
            import torch.distributed._symmetric_memory as symm
            self._bsym = symm.empty(self.K * self.N, dtype=self.dtype, device=self.device)
            grp = self.group if self.group is not None else dist.group.WORLD
            self._hdl = symm.rendezvous(self._bsym, group=grp)
            self._bptrs = [int(p) for p in self._hdl.buffer_ptrs]
            self.Bfull = self._bsym.view(self.K, self.N)
            if self.is_owner:
                self.B = self.Bfull               # the owner's operand IS its replica: nothing to pack
            self.flags = torch.zeros(8, dtype=torch.int32, device=self.device)
            self._side = [torch.cuda.Stream(device=self.device) for _ in range(2)]
            self._ev_go = torch.cuda.Event()
            self._ev_side = [torch.cuda.Event() for _ in self._side]
            return True
        except Exception as e:
            print(f"decx_b200.sharded: symmetric memory unavailable ({type(e).__name__}: {e}); one launch per panel",
                  file=sys.stderr)
            self._hdl = None
            self.bcast = "broadcast"
            return False

    # ------------------------------------------------------------------ "fused": the kernel fetches B itself
    def _setup_fused(self):
        """A full K x N replica of B per rank plus two flag arrays in ONE symmetric allocation (the owner's
        replica is its B); every rank maps every other rank's copy."""
        import sys
        try:
            import torch.distributed._symmetric_memory as symm
            n = self.K * self.N
            self._bsym = symm.empty(n + 128, dtype=self.dtype, device=self.device)     # + 256 bytes of flags
            grp = self.group if self.group is not None else dist.group.WORLD
            self._hdl = symm.rendezvous(self._bsym, group=grp)
            self._bptrs = [int(p) for p in self._hdl.buffer_ptrs]
            self.Bfull = self._bsym[:n].view(self.K, self.N)
            if self.is_owner:
                self.B = self.Bfull
            words = self._bsym[n:].view(torch.int32)
            words.zero_()
            self.flags, self.pub_flags = words[:16], words[16:32]
            self._pub_ptrs = [p + n * self._esz_of(self.dtype) + 64 for p in self._bptrs]
            mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
            self._mc_ptr = mc or None
            self._mc_pub_ptr = (mc + n * self._esz_of(self.dtype) + 64) if mc else None
            if self._scatter == "multicast" and not mc:
                print("decx_b200.sharded: no NVLink multicast mapping for the replica; the owner pushes piece by piece",
                      file=sys.stderr)
                self._scatter = "push"
            return True
        except Exception as e:
            print(f"decx_b200.sharded: symmetric memory unavailable ({type(e).__name__}: {e}); copy-engine delivery",
                  file=sys.stderr)
            self._hdl = None
            return False

    @staticmethod
    def _esz_of(dtype):
        return torch.empty(0, dtype=dtype).element_size()

    def _fused_prepare(self):
        capi = self._capi
        active = [r for r, (_, n) in enumerate(self.rows) if n > 0]
        tuples = fetch_jobs(self.rank, self.owner, active, self.K, self.panels, self._bptrs, self._pub_ptrs,
                            scatter=self._scatter, mc_ptr=self._mc_ptr, mc_pub_ptr=self._mc_pub_ptr)
        self._jobs = [capi.fetch_job(*t) for t in tuples]
        self._pulls = any(t[8] is None for t in tuples)
        need = int(capi.lib.decxb200_fetch_scratch_bytes(max(len(self._jobs), 1)))
        self._fetch_scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        # ranks whose D rows live in the owner's memory forward them through a local ring (see the C header)
        self._d_stage = None
        if self._forward_d is None:
            self._forward_d = self.world == 2
        if self._forward_d and not self.is_owner and self.gather == "peer":
            self._d_stage = torch.empty(int(capi.lib.decxb200_fetch_d_stage_bytes()), dtype=torch.uint8, device=self.device)

    def _fused_gemm(self, epoch, fetch=True):
        if self.nrows == 0:
            return
        G = self._G
        ends = [c0 + w for c0, w in self.panels]
        jobs = self._jobs if fetch else []
        gated = (bool(jobs) and self._pulls) or not self.is_owner
        with torch.cuda.device(self.device):
            G.gemm_fp16_fetch(self.A, self.Bfull, self._d_ptr, self.N, ends, self.flags if gated else None,
                              self.pub_flags if (jobs and self._pulls) else None, epoch, jobs,
                              self._fetch_scratch if jobs else None,
                              status=self.status, max_ctas=self._max_ctas, tile=self._tile,
                              d_stage=self._d_stage if jobs else None)
        self.launches += self._capi.lib.decxb200_last_launch_count()
        self.kernel_variant = self._capi.lib.decxb200_last_kernel_variant()

    def fetch_stats(self):
        """Timing record of the last fused launch on this rank (after a synchronize), in microseconds relative
        to the kernel's start: when each panel was complete, kernel duration, total loader wait."""
        if self.overlap != "fused" or not self._jobs:
            return None
        w = self._fetch_scratch[256:512].view(torch.int64).cpu().tolist()
        t0 = w[16]
        return {"panel_ready_us": [round((w[i] - t0) / 1e3, 1) if w[i] else None for i in range(len(self.panels))],
                "scatter_piece_us": [round((w[24 + i] - t0) / 1e3, 1) if w[24 + i] else None for i in range(min(8, len(self.panels)))],
                "kernel_us": round((w[17] - t0) / 1e3, 1), "loader_wait_us_sum": round(w[18] / 1e3, 1),
                "loader_waits": w[19]}

    def _deliver_replica(self, epoch):
        """Communication stream of the "single" overlap: fill this rank's replica of B panel by panel and flag
        each panel.  Every rank pulls its row block of the panel from the owner, then the other row blocks from
        the ranks that hold them; copy engines only, ordered by symmetric-memory stream barriers."""
        G, st = self._G, self.comm_stream
        esz, N, rows = self._esz, self.N, self.K // self.world
        pitch = N * esz
        self._hdl.barrier(channel=0)                       # the owner's B is final; nobody still reads old data
        for j, (c0, w) in enumerate(self.panels):
            if self.is_owner:
                G.write_flag(self.flags, j, epoch, st)     # the owner holds every panel already
                self._hdl.barrier(channel=1)
                continue
            mine = (self.rank * rows * N + c0) * esz
            G.copy2d(self._bptrs[self.rank] + mine, pitch, self._bptrs[self.owner] + mine, pitch, w * esz, rows, st)
            self._hdl.barrier(channel=1)                   # every rank holds its own row block of panel j
            # the other row blocks, each in two halves, dealt over several streams: one stream's copies run one
            # after the other on one copy engine, and a single engine pulling from peers is far below link speed
            self._ev_go.record(st)
            for side in self._side:
                side.wait_event(self._ev_go)
            lanes, k = [st] + self._side, 0
            half = rows // 2
            for d in range(1, self.world):
                src = (self.rank + d) % self.world
                for r0, nr in ((0, half), (half, rows - half)):
                    if nr == 0:
                        continue
                    off = ((src * rows + r0) * N + c0) * esz
                    k += 1
                    G.copy2d(self._bptrs[self.rank] + off, pitch, self._bptrs[src] + off, pitch, w * esz, nr,
                             lanes[k % len(lanes)])
            for side, ev in zip(self._side, self._ev_side):
                ev.record(side)
                st.wait_event(ev)
            G.write_flag(self.flags, j, epoch, st)

    def _single_gemm(self, epoch):
        if self.nrows == 0:
            return
        ends = [c0 + w for c0, w in self.panels]
        arr = (ctypes.c_uint32 * len(ends))(*ends)
        capi = self._capi
        capi.check(capi.lib.decxb200_gemm_fp16_panels(
            torch.cuda.current_stream(self.device).cuda_stream, self.nrows, self.N, self.K,
            self.A.data_ptr(), self.A.stride(0), self.Bfull.data_ptr(), self.N, self._d_ptr, self.N,
            self.status.data_ptr(), len(ends), arr, self.flags.data_ptr(), epoch, self._max_ctas, self._tile))
        self.launches += capi.lib.decxb200_last_launch_count()
        self.kernel_variant = capi.lib.decxb200_last_kernel_variant()

    def compute_only(self):
        """This rank's GEMM launch(es) with B already in place and no communication (for kernel timing)."""
        self.launches = 0
        if self.overlap == "fused":
            self._fused_gemm(self._epoch, fetch=False)     # the replica and its flags hold this epoch
        elif self.overlap == "single":
            self._single_gemm(self._epoch)                 # the flags already hold this epoch
        else:
            for j in range(len(self.panels)):
                self._panel_gemm(j)
        return self.launches

    def _send_panel_p2p(self, j):
        c0, w = self.panels[j]
        buf, rows = self.Bp[j], self.K // self.world
        blk, base = rows * w, self._poff[j]
        if self.is_owner:
            buf.copy_(self.B[:, c0:c0 + w])
        self._hdl.barrier(channel=0)                       # the owner's copy of the panel is complete
        if not self.is_owner:
            lo = base + self.rank * blk
            self._bsym[lo:lo + blk].copy_(self._peer[self.owner][lo:lo + blk])
        self._hdl.barrier(channel=1)                       # every rank holds its own row block
        if not self.is_owner:
            for d in range(1, self.world):
                src = (self.rank + d) % self.world         # stagger the sources over the ranks
                lo = base + src * blk
                self._bsym[lo:lo + blk].copy_(self._peer[src][lo:lo + blk])

    # ------------------------------------------------------------------ peer-visible D on the owner
    def _setup_peer_d(self):
        capi = self._capi
        handle = torch.zeros(64, dtype=torch.uint8)
        with torch.cuda.device(self.device):
            if self.is_owner:
                p = ctypes.c_void_p()
                capi.check(capi.lib.decxb200_ipc_alloc(self.M * self.N * self._esz, ctypes.byref(p)))
                self._owned = p.value
                buf = ctypes.create_string_buffer(64)
                capi.check(capi.lib.decxb200_ipc_export(p.value, buf))
                handle = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
            h = handle.to(self.device)
            dist.broadcast(h, src=self.owner, group=self.group)
            if self.is_owner:
                base = self._owned
                self.D = torch.as_tensor(_RawCuda(base, (self.M, self.N), _TYPESTR[self.dtype]), device=self.device)
            else:
                p = ctypes.c_void_p()
                capi.check(capi.lib.decxb200_ipc_open(bytes(h.cpu().numpy().tobytes()), ctypes.byref(p)))
                self._peer_base = base = p.value
                self.D = None
            self._d_ptr = base + self.row0 * self.N * self._esz

    def close(self):
        if self.on_gpu:
            torch.cuda.synchronize(self.device)
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
        self._peer = None
        self._hdl = None
        if self._peer_base is not None:
            self._capi.lib.decxb200_ipc_close(self._peer_base)
            self._peer_base = None
        if self._owned is not None:
            self.D = None
            self._capi.lib.decxb200_ipc_free(self._owned)
            self._owned = None

    # ------------------------------------------------------------------ one step
    def _panel_gemm(self, j):
        c0, w = self.panels[j]
        if self.nrows == 0:
            return
        if self.gemm_fn is not None:
            self.gemm_fn(self.A, self.Bp[j], self.D_local[:, c0:c0 + w])
            return
        G = self._G
        if self.gather == "peer":
            d_ptr = self._d_ptr + c0 * self._esz
        else:
            d_ptr = self.D_local.data_ptr() + c0 * self._esz
        ldb = self.Bp[j].stride(0)
        self.launches += G.gemm_raw(self._dt, self.nrows, w, self.K, self.A.data_ptr(), self.A.stride(0),
                                    self.Bp[j].data_ptr() + (c0 * self._esz if self.world == 1 else 0), ldb,
                                    None, 0, d_ptr, self.N,
                                    ws_ptr=self.workspace.data_ptr() if self._ws_bytes else None,
                                    ws_bytes=self._ws_bytes, status_ptr=self.status.data_ptr(),
                                    stream=torch.cuda.current_stream(self.device).cuda_stream,
                                    max_ctas=self._max_ctas)

    def _send_panel(self, j):
        """Make panel j of B present on every rank (issued on the communication stream)."""
        if self.bcast == "p2p":
            return self._send_panel_p2p(j)
        c0, w = self.panels[j]
        buf = self.Bp[j]
        if self.is_owner:
            buf.copy_(self.B[:, c0:c0 + w])
        if self.bcast == "scatter_allgather" and self.K % self.world == 0:
            rows = self.K // self.world
            mine = buf[self.rank * rows:(self.rank + 1) * rows]
            if self.is_owner:
                chunks = [buf[r * rows:(r + 1) * rows] for r in range(self.world)]
                dist.scatter(mine, scatter_list=chunks, src=self.owner, group=self.group)
            else:
                dist.scatter(mine, src=self.owner, group=self.group)
            dist.all_gather_into_tensor(buf, mine, group=self.group)     # in place: `mine` is this rank's slice
        else:
            dist.broadcast(buf, src=self.owner, group=self.group)

    def step(self):
        """Broadcast B, multiply, gather on the owner.  Asynchronous on a GPU: the caller synchronises."""
        self.launches = 0
        if self.world == 1:
            self.Bp = [self.B]
            self._panel_gemm(0)
            return
        if self.overlap == "fused":
            with torch.cuda.device(self.device):
                self._epoch += 1
                self._hdl.barrier(channel=0)               # B is final on the owner; nobody still reads the old replicas
                self._fused_gemm(self._epoch)
                self._hdl.barrier(channel=1)               # every rank's rows have reached the owner
            return
        if self.overlap == "single":
            with torch.cuda.device(self.device):
                cur = torch.cuda.current_stream(self.device)
                self._epoch += 1
                self.comm_stream.wait_stream(cur)          # the previous step no longer reads the replica
                with torch.cuda.stream(self.comm_stream):
                    self._deliver_replica(self._epoch)
                self._single_gemm(self._epoch)             # waits on the panel flags inside the kernel
                dist.barrier(group=self.group)             # every rank's rows have reached the owner
                cur.wait_stream(self.comm_stream)
            return
        if self.on_gpu:
            with torch.cuda.device(self.device):
                cur = torch.cuda.current_stream(self.device)
                self.comm_stream.wait_stream(cur)
                with torch.cuda.stream(self.comm_stream):
                    for j in range(len(self.panels)):
                        self._send_panel(j)
                        self.events[j].record(self.comm_stream)
                for j in range(len(self.panels)):
                    cur.wait_event(self.events[j])
                    self._panel_gemm(j)
                if self.gather == "collective":
                    self._collect()
                dist.barrier(group=self.group)      # every rank's rows have reached the owner
        else:
            for j in range(len(self.panels)):
                self._send_panel(j)
                self._panel_gemm(j)
            self._collect()
            dist.barrier(group=self.group)

    def _collect(self):
        """Mode "collective": full-width row blocks are contiguous in the owner's D, one message per rank."""
        if self.is_owner:
            reqs = []
            for r, (r0, n) in enumerate(self.rows):
                if r != self.owner and n > 0:
                    reqs.append(dist.irecv(self.D[r0:r0 + n], src=r, group=self.group))
            for q in reqs:
                q.wait()
        elif self.nrows > 0:
            dist.send(self.D_local, dst=self.owner, group=self.group)
