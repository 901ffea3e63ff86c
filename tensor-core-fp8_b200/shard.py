"""N-sharded multi-GPU plan for one large GEMM.

C's columns are independent and B is stored as N rows of K bytes, so a column block of
B / C is a contiguous row slab of B's storage: rank r of R owns rows
[n_begin, n_end) of B and the same columns of C; A is replicated.  The compute step
exchanges nothing.  An all-gather of the C blocks is optional and timed separately.
(The reference has no multi-GPU code; its operator, GEMM/include/gemm.cuh:12-55, is
what each rank calls on its shard.)
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    n_begin: int
    n_end: int

    @property
    def n(self) -> int:
        return self.n_end - self.n_begin


def column_shard(n: int, rank: int, world: int, align: int = 256) -> Shard:
    """Even split of N columns in units of `align` (the widest tile), remainder to the low ranks."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    units = (n + align - 1) // align
    base, extra = divmod(units, world)
    begin_u = rank * base + min(rank, extra)
    end_u = begin_u + base + (1 if rank < extra else 0)
    return Shard(rank, world, min(n, begin_u * align), min(n, end_u * align))


def all_shards(n: int, world: int, align: int = 256):
    return [column_shard(n, r, world, align) for r in range(world)]


def gather_layout_to_row_major(blocks, m: int):
    """All-gather returns [R][M][N/R]; this is the index map back to row-major [M][N] (host-side check)."""
    import torch
    return torch.cat([b.reshape(m, -1) for b in blocks], dim=1)


class _DevicePointer:
    """Lets torch wrap a raw device pointer (``torch.as_tensor``) without owning it."""

    def __init__(self, ptr: int, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 2}


class SharedC:
    """The full M x N matrix C of every rank, visible to every rank (one process per GPU, one node).

    Each rank allocates its own full C through the library's CUDA-IPC helpers and hands the handle to
    the others over `torch.distributed`; each rank opens its peers' handles with its own device current,
    so the mappings (and peer access) belong to the device whose kernels will store through them.
    `tensors[r]` is rank r's C as seen from this process.  Before first use the mapping is proven with
    plain copies: every rank writes its rank number into one word of every matrix and checks its own.
    Call `close()` (collective) when done.
    """

    def __init__(self, m: int, n_total: int, device, group=None, multicast: bool = False):
        import ctypes
        import torch
        import torch.distributed as dist
        from . import _cabi
        lib = _cabi.lib()
        self._lib, self._group = lib, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("fused all-gather covers one box of at most 8 GPUs")
        if n_total < self.world:
            raise ValueError("need at least one column per rank")
        self.device = torch.device(device)
        self._ptrs = [None] * self.world
        self.multicast_ptr = 0
        self._symm = None
        if multicast:
            # NVSwitch multicast: torch's symmetric memory allocates the matrices, exchanges the handles and
            # binds them to one multicast address (needs an NCCL-capable process group on this device)
            import torch.distributed._symmetric_memory as symm_mem
            with torch.cuda.device(self.device):
                self.own = symm_mem.empty((m, n_total), dtype=torch.float32, device=self.device)
                self._symm = symm_mem.rendezvous(self.own, group if group is not None else dist.group.WORLD)
                if not self._symm.multicast_ptr:
                    raise RuntimeError("this system offers no NVLink multicast for symmetric memory")
                self.multicast_ptr = int(self._symm.multicast_ptr)
                self._ptrs = [int(p) for p in self._symm.buffer_ptrs]
                self.tensors = [self.own if r == self.rank else self._symm.get_buffer(r, (m, n_total), torch.float32)
                                for r in range(self.world)]
                self._check_mappings(torch, dist, group)
            return
        with torch.cuda.device(self.device):
            own = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            _cabi.check(lib.b200fp8_ipc_alloc(m * n_total * 4, ctypes.byref(own), handle), "ipc_alloc")
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    self._ptrs[r] = own.value
                else:
                    p = ctypes.c_void_p()
                    _cabi.check(lib.b200fp8_ipc_open(h, ctypes.byref(p)), f"ipc_open of rank {r}'s C")
                    self._ptrs[r] = p.value
            self.tensors = [torch.as_tensor(_DevicePointer(p, (m, n_total)), device=self.device) for p in self._ptrs]
            self.own = self.tensors[self.rank]
            self._check_mappings(torch, dist, group)

    def _check_mappings(self, torch, dist, group):
        # prove every mapping with copies (a bad mapping fails here with an error, not inside a kernel)
        mark = torch.full((1,), float(self.rank + 1), dtype=torch.float32, device=self.device)
        for t in self.tensors:
            t[0, self.rank:self.rank + 1].copy_(mark)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        seen = self.own[0, :self.world].cpu().tolist()
        if seen != [float(r + 1) for r in range(self.world)]:
            raise RuntimeError(f"peer mapping check failed on rank {self.rank}: {seen}")
        dist.barrier(group=group)

    def pointers(self):
        import ctypes
        return (ctypes.c_void_p * self.world)(*self._ptrs)

    def close(self):
        """Collective: unmap the peers' matrices, then free the own one."""
        import torch
        import torch.distributed as dist
        if self._ptrs is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self._group)
        if self._symm is not None:                    # torch owns the symmetric allocation and its multicast binding
            self.tensors, self._ptrs = None, None
            dist.barrier(group=self._group)
            return
        self.tensors, self.own = None, None
        with torch.cuda.device(self.device):
            for r, p in enumerate(self._ptrs):
                if r != self.rank:
                    self._lib.b200fp8_ipc_close(p)
            dist.barrier(group=self._group)
            self._lib.b200fp8_ipc_free(self._ptrs[self.rank])
        self._ptrs = None


def gemm_allgather(a, b_shard, shared: "SharedC", shard: Shard, n_total: int, *, depth: int = 0, kernel: int = 0):
    """This rank's column block of C = A B^T, written into every rank's full C by the kernel's epilogue."""
    import ctypes
    import torch
    from . import _cabi
    from .gemm import dtype_code
    m, k = a.shape
    opt = _cabi.Options(ctypes.sizeof(_cabi.Options), depth, kernel, 0, 0)
    with torch.cuda.device(a.device):
        rc = _cabi.lib().b200fp8_gemm_rowcol_f32_allgather(
            m, k, shard.n, a.data_ptr(), dtype_code(a), b_shard.data_ptr(), dtype_code(b_shard), shared.pointers(),
            shared.multicast_ptr or None, shared.world, shared.rank, n_total, shard.n_begin, ctypes.byref(opt),
            torch.cuda.current_stream(a.device).cuda_stream)
    _cabi.check(rc, "gemm_allgather")


class HostShardedGemm:
    """End to end from HOST buffers on R GPUs: what `b200fp8_gemm_rowcol_f32_host` does on one.

    Uploading the replicated A once per rank would push R copies of it through the host's PCIe complex, so every
    rank uploads only its M/R rows of A (and its own rows of B) and the ranks hand their rows to each other over
    NVLink.  The phases overlap: uploads run on a copy stream; rank j's rows travel as broadcast j on a
    communication stream; the operator runs in row blocks, the own block first (it needs no communication) and
    block j as soon as broadcast j has landed; each finished block of C goes down on a third stream while the next
    block computes.  The own rows do not wait for the whole B shard either: B goes up in `col_blocks` pieces and the
    own rows are multiplied with each piece as it lands, the finished column block of C leaving at once (a pitched
    copy), so that the download -- which bounds the call -- starts after a fraction of the uploads.  `__call__(a_rows_host, b_shard_host, c_shard_host)`: pinned host tensors holding this rank's M/R
    rows of A, its rows of B and room for its M x n column block of C; returns when the block is complete in host
    memory.  With `breakdown=True` it also returns the milliseconds, from the call's start, at which each phase
    ended on the device.
    """

    def __init__(self, m: int, k: int, shard: Shard, a_dtype, b_dtype, device, group=None, row_blocks: int = 8,
                 col_blocks: int = 4):
        import torch
        import torch.distributed as dist
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if m % self.world:
            raise ValueError("M must be divisible by the number of ranks")
        self.m, self.k, self.shard, self.device = m, k, shard, torch.device(device)
        self.rows_own = m // self.world
        self.a = torch.empty((m, k), dtype=a_dtype, device=self.device)
        self.b = torch.empty((shard.n, k), dtype=b_dtype, device=self.device)
        self.c = torch.empty((m, shard.n), dtype=torch.float32, device=self.device)
        # row blocks of the operator: every rank's rows of A in `sub` pieces, so that about `row_blocks` downloads overlap
        sub = max(1, row_blocks // self.world)
        step = -(-self.rows_own // sub)
        step = -(-step // 256) * 256
        self.blocks = {j: [(j * self.rows_own + r0, min((j + 1) * self.rows_own, j * self.rows_own + r0 + step))
                           for r0 in range(0, self.rows_own, step)] for j in range(self.world)}
        # column pieces of the B shard for the own rows (multiples of 256 columns; one piece if the shard is narrow)
        cstep = -(-shard.n // max(1, col_blocks))
        cstep = max(256, -(-cstep // 256) * 256)
        self.col_pieces = [(c0, min(shard.n, c0 + cstep)) for c0 in range(0, shard.n, cstep)]
        self.copy_in = torch.cuda.Stream(device=self.device)
        self.comm = torch.cuda.Stream(device=self.device)
        self.copy_out = torch.cuda.Stream(device=self.device)

    def __call__(self, a_rows_host, b_shard_host, c_shard_host, *, depth: int = 0, kernel: int = 0, breakdown: bool = False):
        import torch
        import torch.distributed as dist
        from . import gemm as g
        ev = lambda: torch.cuda.Event(enable_timing=breakdown)
        cur = torch.cuda.current_stream(self.device)
        start, up_a, up_b, last_bcast, first_gemm, last_gemm, last_down = ev(), ev(), ev(), ev(), ev(), ev(), ev()
        start.record(cur)
        r0 = self.rank * self.rows_own
        own = self.a[r0:r0 + self.rows_own]
        self.copy_in.wait_stream(cur)
        piece_up = []
        with torch.cuda.stream(self.copy_in):
            own.view(torch.uint8).copy_(a_rows_host.view(torch.uint8), non_blocking=True)
            up_a.record(self.copy_in)
            for (c0, c1) in self.col_pieces:             # rows c0..c1 of the shard = columns c0..c1 of this rank's C
                self.b[c0:c1].view(torch.uint8).copy_(b_shard_host[c0:c1].view(torch.uint8), non_blocking=True)
                piece_up.append(torch.cuda.Event())
                piece_up[-1].record(self.copy_in)
            up_b.record(self.copy_in)
        arrived = {}
        if self.world > 1:
            self.comm.wait_event(up_a)                       # rank j's broadcast sends rows that its upload wrote
            with torch.cuda.stream(self.comm):
                for j in range(self.world):                  # same order on every rank: broadcast j carries rank j's rows
                    rows = self.a[j * self.rows_own:(j + 1) * self.rows_own]
                    dist.broadcast(rows.view(torch.uint8), src=dist.get_global_rank(self.group, j) if self.group is not None else j,
                                   group=self.group)
                    arrived[j] = torch.cuda.Event()
                    arrived[j].record(self.comm)
                last_bcast.record(self.comm)
        else:
            last_bcast.record(cur)
        cur.wait_event(up_a)
        first = True
        from . import _cabi
        lib = _cabi.lib()
        n = self.shard.n
        # own rows: column piece by column piece, each as soon as its rows of B are on the device
        for p, (c0, c1) in enumerate(self.col_pieces):
            cur.wait_event(piece_up[p])
            for (lo, hi) in self.blocks[self.rank]:
                g.gemm_ex(self.a[lo:hi], self.b[c0:c1], self.c[lo:hi, c0:c1], depth=depth, kernel=kernel)
                done = torch.cuda.Event()
                done.record(cur)
                if first:
                    first_gemm.record(cur)
                    first = False
                self.copy_out.wait_event(done)
                dst = c_shard_host.data_ptr() + (lo * n + c0) * 4
                src = self.c.data_ptr() + (lo * n + c0) * 4
                with torch.cuda.device(self.device):
                    _cabi.check(lib.b200fp8_copy_2d_async(dst, n * 4, src, n * 4, (c1 - c0) * 4, hi - lo,
                                                          self.copy_out.cuda_stream), "copy_2d_async")
        # the other ranks' rows: the whole shard is up by now (the last piece's event has been waited for)
        for j in (j for j in range(self.world) if j != self.rank):
            cur.wait_event(arrived[j])
            for (lo, hi) in self.blocks[j]:
                g.gemm_ex(self.a[lo:hi], self.b, self.c[lo:hi], depth=depth, kernel=kernel)
                done = torch.cuda.Event()
                done.record(cur)
                self.copy_out.wait_event(done)
                with torch.cuda.stream(self.copy_out):
                    c_shard_host[lo:hi].copy_(self.c[lo:hi], non_blocking=True)
        last_gemm.record(cur)
        last_down.record(self.copy_out)
        self.copy_out.synchronize()
        self.comm.synchronize()
        cur.synchronize()
        if not breakdown:
            return None
        return {"upload_a_rows": start.elapsed_time(up_a), "upload_b_shard": start.elapsed_time(up_b),
                "a_rows_from_all_ranks": start.elapsed_time(last_bcast), "first_row_block_computed": start.elapsed_time(first_gemm),
                "last_row_block_computed": start.elapsed_time(last_gemm), "last_c_block_in_host_memory": start.elapsed_time(last_down)}


class MultiGpuPlan:
    """The N-sharded GEMM over several GPUs from ONE process: a thin caller of the C ABI's `b200fp8_multi_*` plan,
    which owns the shards' buffers, their streams and one host thread per shard.  `devices` lists the CUDA device of
    every shard (a device may repeat: several shards on one GPU).  With `gather` the kernels' epilogues leave the full
    row-major C on every device."""

    def __init__(self, devices, m: int, k: int, n: int, a_dtype: int = 0, b_dtype: int = 0, gather: bool = False):
        import ctypes
        from . import _cabi
        self._lib, self._ct = _cabi.lib(), ctypes
        self.m, self.k, self.n, self.world, self.gather = m, k, n, len(devices), bool(gather)
        arr = (ctypes.c_int * len(devices))(*devices)
        self._plan = ctypes.c_void_p()
        _cabi.check(self._lib.b200fp8_multi_create(len(devices), arr, m, k, n, a_dtype, b_dtype, 1 if gather else 0,
                                                   ctypes.byref(self._plan)), "multi_create")

    def shard(self, i: int):
        """(device, n_begin, n_end, a_ptr, b_ptr, c_ptr, ldc) of shard i; the pointers are device addresses."""
        ct = self._ct
        dev, nb, ne, ldc = ct.c_int(), ct.c_longlong(), ct.c_longlong(), ct.c_longlong()
        a, b, c = ct.c_void_p(), ct.c_void_p(), ct.c_void_p()
        from . import _cabi
        _cabi.check(self._lib.b200fp8_multi_shard(self._plan, i, ct.byref(dev), ct.byref(nb), ct.byref(ne), ct.byref(a), ct.byref(b),
                                                  ct.byref(c), ct.byref(ldc)), "multi_shard")
        return dev.value, nb.value, ne.value, a.value, b.value, c.value, ldc.value

    def upload(self, a_host, b_host):
        from . import _cabi
        shapes_ok = tuple(a_host.shape) == (self.m, self.k) and tuple(b_host.shape) == (self.n, self.k)
        if a_host.is_cuda or b_host.is_cuda or not shapes_ok or not (a_host.is_contiguous() and b_host.is_contiguous()):
            raise ValueError("upload takes contiguous HOST matrices a [M][K] and b [N][K]")
        _cabi.check(self._lib.b200fp8_multi_upload(self._plan, a_host.data_ptr(), b_host.data_ptr()), "multi_upload")

    def fill_normal(self, sigma_a: float, seed_a: int, sigma_b: float, seed_b: int):
        from . import _cabi
        _cabi.check(self._lib.b200fp8_multi_fill_normal(self._plan, float(sigma_a), int(seed_a), float(sigma_b), int(seed_b)),
                    "multi_fill_normal")

    def run(self, steps: int = 1, *, depth: int = 0, kernel: int = 0) -> float:
        """`steps` operator calls per shard, all shards at once; returns the maximum over the shards of ms per step."""
        from . import _cabi
        ct = self._ct
        opt = _cabi.Options(ct.sizeof(_cabi.Options), depth, kernel, 0, 0)
        ms = ct.c_float(0)
        _cabi.check(self._lib.b200fp8_multi_run(self._plan, steps, ct.byref(opt), ct.byref(ms)), "multi_run")
        return ms.value

    def download(self, c_host, from_shard: int = 0):
        import torch
        from . import _cabi
        if c_host.is_cuda or c_host.dtype != torch.float32 or tuple(c_host.shape) != (self.m, self.n) or not c_host.is_contiguous():
            raise ValueError("download takes a contiguous HOST float32 matrix [M][N]")
        _cabi.check(self._lib.b200fp8_multi_download(self._plan, c_host.data_ptr(), from_shard), "multi_download")
        return c_host

    def close(self):
        if self._plan:
            self._lib.b200fp8_multi_destroy(self._plan)
            self._plan = self._ct.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
