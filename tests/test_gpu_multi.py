"""The column-sharded forward on two GPUs: through ShardedNf4Linear (torch.distributed, NCCL) and
through nf4_sharded_linear_forward_dev with a raw two-rank NCCL communicator.  Every rank compares
the gathered output with its own unsharded forward of the full weight.  Skipped on a machine with
fewer than two GPUs (the host logic is covered on CPU by tests/test_sharded_gloo.py)."""
import ctypes
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _NcclId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


def _worker(rank, world, port, results):
    import torch.distributed as dist

    from unifur_b200 import _lib
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward
    from unifur_b200.sharded import ShardedNf4Linear

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = True
    try:
        L = _lib.load()
        for case, (m, k, n, r, gran) in enumerate(((8, 3584, 512, 16, 64), (300, 1024, 1536, 64, 64),
                                                   (4, 512, 320, 8, 64))):
            g = torch.Generator(device=dev).manual_seed(40 + case)  # the same weight on every rank
            w = torch.randn(n * k, device=dev, generator=g) * 0.02
            full = PackedNf4Tensor.quantize(w)
            la = (torch.randn(r, k, device=dev, generator=g) * 0.01).bfloat16()
            lb = (torch.randn(n, r, device=dev, generator=g) * 0.01).bfloat16()
            x = torch.randn(m, k, device=dev, generator=g).bfloat16()
            y_full = linear_forward(x, full, k, n, _lib.LAYOUT_OUT_IN, lora_a=la, lora_b=lb, lora_scale=2.0)
            lin = ShardedNf4Linear.from_full(full, k, n, world, rank, lora_a=la, lora_b=lb, lora_scale=2.0,
                                             granule=gran)
            y1 = lin.forward(x)                      # allocating form
            plan = lin.plan(x)
            y2 = plan.run().clone()                  # preallocated form
            torch.cuda.synchronize()
            tol = y_full.float().abs() * 2.0 ** -7 + 4e-6 * float(y_full.float().abs().max())
            c1 = bool(((y1.float() - y_full.float()).abs() <= tol).all())
            # the decode kernel is deterministic; the prefill pre-pass meets its partial sums through
            # shared-memory adds whose order is not fixed, so two runs may differ in a last bit
            c2 = torch.equal(y1, y2) if m <= 16 else bool(((y1.float() - y2.float()).abs() <= tol).all())
            if not (c1 and c2):
                print(f"rank {rank} case {case}: within tolerance {c1}, plan equals forward {c2}", flush=True)
            ok &= c1 and c2
        # the same exchange below the C ABI: raw NCCL communicator, equal shards
        nccl = ctypes.CDLL(os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "nccl", "lib",
                                        "libnccl.so.2"), mode=ctypes.RTLD_GLOBAL)
        uid = _NcclId()
        buf = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            assert nccl.ncclGetUniqueId(ctypes.byref(uid)) == 0
            buf.copy_(torch.frombuffer(bytearray(bytes(uid.internal)), dtype=torch.uint8))
        dist.broadcast(buf, 0)
        ctypes.memmove(ctypes.byref(uid), bytes(buf.cpu().numpy().tobytes()), 128)
        comm = ctypes.c_void_p()
        nccl.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _NcclId, ctypes.c_int]
        assert nccl.ncclCommInitRank(ctypes.byref(comm), world, uid, rank) == 0
        m, k, n, r = 16, 4096, 1024, 16
        nl = n // world
        g = torch.Generator(device=dev).manual_seed(99)
        w = torch.randn(n * k, device=dev, generator=g) * 0.02
        full = PackedNf4Tensor.quantize(w)
        la = (torch.randn(r, k, device=dev, generator=g) * 0.01).bfloat16()
        lb = (torch.randn(n, r, device=dev, generator=g) * 0.01).bfloat16()
        x = torch.randn(m, k, device=dev, generator=g).bfloat16()
        y_ref = linear_forward(x, full, k, n, _lib.LAYOUT_OUT_IN, lora_a=la, lora_b=lb, lora_scale=2.0)
        codes = full.codes[rank * nl * (k // 2):(rank + 1) * nl * (k // 2)].contiguous()
        absmax = full.absmax[rank * nl * (k // 64):(rank + 1) * nl * (k // 64)].contiguous()
        lb_l = lb[rank * nl:(rank + 1) * nl].contiguous()
        slab = torch.zeros(m, nl, dtype=torch.bfloat16, device=dev)
        y_out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
        gb = int(L.nf4_sharded_gather_bytes(m, nl, world, _lib.DTYPE_BF16, 0))
        gbuf = torch.zeros(gb, dtype=torch.uint8, device=dev)
        ws = torch.zeros(max(int(L.nf4_linear_workspace_bytes(m, k, nl, r)), 256), dtype=torch.uint8, device=dev)
        a = _lib.LinearArgs()
        a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
        a.rows, a.d_in, a.d_out = m, k, nl
        a.x, a.packed, a.absmax = x.data_ptr(), codes.data_ptr(), absmax.data_ptr()
        a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb_l.data_ptr(), r, 2.0
        a.y, a.ldy = slab.data_ptr(), nl
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        vp = ctypes.c_void_p
        _lib.check(L.nf4_sharded_linear_forward_dev(ctypes.byref(a), comm, rank, world, vp(gbuf.data_ptr()), gb,
                                                    vp(y_out.data_ptr()), n, None))
        torch.cuda.synchronize()
        c3 = torch.equal(y_out, y_ref)   # the decode kernel's arithmetic per row does not depend on the shard
        if not c3:
            print(f"rank {rank}: C ABI gather differs, max abs diff "
                  f"{(y_out.float() - y_ref.float()).abs().max().item()}", flush=True)
        ok &= c3
        nccl.ncclCommDestroy(comm)
    finally:
        results[rank] = 1 if ok else 0
        dist.barrier()
        dist.destroy_process_group()


def _scatter_worker(rank, world, port, results):
    """Every rank's decode kernel stores its columns into every rank's output (peer stores through
    IPC-mapped buffers, arrival counters, the bounded wait kernel); no collective on the data path."""
    import torch.distributed as dist

    from unifur_b200 import _lib
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward
    from unifur_b200.sharded import map_peer_tensors

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = True
    peers_y = peers_c = peers_z = None
    try:
        L = _lib.load()
        k, n, r = 4096, 1024, 16
        nl = n // world
        rows_max = 16
        y_mine = torch.zeros(rows_max, n, dtype=torch.bfloat16, device=dev)
        cnt_mine = torch.zeros(64, dtype=torch.int32, device=dev)
        peers_y = map_peer_tensors(y_mine)     # every rank's output and counters, mapped into this GPU
        peers_c = map_peer_tensors(cnt_mine)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.Generator(device=dev).manual_seed(123)     # the same layer on every rank
        w = torch.randn(n * k, device=dev, generator=g) * 0.02
        full = PackedNf4Tensor.quantize(w)
        la = (torch.randn(r, k, device=dev, generator=g) * 0.01).bfloat16()
        lb = (torch.randn(n, r, device=dev, generator=g) * 0.01).bfloat16()
        codes = full.codes[rank * nl * (k // 2):(rank + 1) * nl * (k // 2)].contiguous()
        absmax = full.absmax[rank * nl * (k // 64):(rank + 1) * nl * (k // 64)].contiguous()
        lb_l = lb[rank * nl:(rank + 1) * nl].contiguous()
        # a second layer that reads the first one's gathered output: [n2, n], sharded the same way
        n2 = 512
        nl2 = n2 // world
        w2 = torch.randn(n2 * n, device=dev, generator=g) * 0.02
        full2 = PackedNf4Tensor.quantize(w2)
        codes2 = full2.codes[rank * nl2 * (n // 2):(rank + 1) * nl2 * (n // 2)].contiguous()
        absmax2 = full2.absmax[rank * nl2 * (n // 64):(rank + 1) * nl2 * (n // 64)].contiguous()
        z_mine = torch.zeros(rows_max, n2, dtype=torch.bfloat16, device=dev)
        peers_z = map_peer_tensors(z_mine)

        def shard_args(m, x_t, d_in, d_out_l, codes_t, absmax_t, rank_r):
            ws = torch.zeros(max(int(L.nf4_linear_workspace_bytes(m, d_in, d_out_l, rank_r)), 256), dtype=torch.uint8,
                             device=dev)
            a = _lib.LinearArgs()
            a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
            a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
            a.rows, a.d_in, a.d_out = m, d_in, d_out_l
            a.x, a.packed, a.absmax = x_t.data_ptr(), codes_t.data_ptr(), absmax_t.data_ptr()
            if rank_r:
                a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb_l.data_ptr(), rank_r, 2.0
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            return a, ws

        def outputs(peers, counter_index, ldy, signal, wait_index=None):
            po = _lib.PeerOutputs()
            po.struct_bytes = ctypes.sizeof(_lib.PeerOutputs)
            po.world, po.rank, po.ldy_full = world, rank, ldy
            for i in range(world):
                po.y_full[i] = peers[i].data_ptr()
                po.arrivals[i] = peers_c[i][counter_index:counter_index + 1].data_ptr()
            po.signal = 1 if signal else 0
            if wait_index is not None:
                po.wait_arrivals = cnt_mine[wait_index:wait_index + 1].data_ptr()
                po.wait_expected = world
            return po

        for m in (1, 8, 16):
            x = torch.randn(m, k, device=dev, generator=g).bfloat16()
            y_ref = linear_forward(x, full, k, n, _lib.LAYOUT_OUT_IN, lora_a=la, lora_b=lb, lora_scale=2.0)
            z_ref = linear_forward(y_ref, full2, n, n2, _lib.LAYOUT_OUT_IN)
            a1, ws1 = shard_args(m, x, k, nl, codes, absmax, r)
            a2, ws2 = shard_args(m, y_mine, n, nl2, codes2, absmax2, 0)   # x of layer 2 = this rank's gathered y
            po1 = outputs(peers_y, 0, n, signal=True)
            po2 = outputs(peers_z, 1, n2, signal=True, wait_index=0)       # waits for layer 1's arrivals in the kernel
            for _rep in range(3):  # the counters come back to zero every time
                y_mine.zero_()
                z_mine.zero_()
                torch.cuda.synchronize()
                dist.barrier()      # nobody writes into an output that is still being cleared
                _lib.check(L.nf4_linear_forward_scatter_dev(ctypes.byref(a1), ctypes.byref(po1), None))
                _lib.check(L.nf4_linear_forward_scatter_dev(ctypes.byref(a2), ctypes.byref(po2), None))
                _lib.check(L.nf4_peer_arrivals_wait_dev(ctypes.c_void_p(cnt_mine[1:2].data_ptr()), world,
                                                        2_000_000_000, None))
                torch.cuda.synchronize()
                good = (torch.equal(y_mine[:m], y_ref) and torch.equal(z_mine[:m], z_ref)
                        and int(cnt_mine[0].item()) == 0 and int(cnt_mine[1].item()) == 0)
                if not good:
                    print(f"rank {rank} m {m}: layer 1 equal {torch.equal(y_mine[:m], y_ref)}, layer 2 equal "
                          f"{torch.equal(z_mine[:m], z_ref)}, counters {cnt_mine[:2].tolist()}", flush=True)
                ok &= good
                dist.barrier()      # everyone has compared before the next round overwrites
        # the same through ShardedNf4Linear.peer_store_plan: a shape of the tensor-core kernel (the
        # forward writes its columns in place, a second kernel pushes them to the peers) and a
        # decode shape (the kernel's own epilogue stores into the peers)
        from unifur_b200.sharded import ShardedNf4Linear

        for case, (m3, k3, n3, r3) in enumerate(((300, 1024, 1536, 64), (8, 3584, 512, 16), (2048, 512, 256, 0))):
            g3 = torch.Generator(device=dev).manual_seed(777 + case)
            full3 = PackedNf4Tensor.quantize(torch.randn(n3 * k3, device=dev, generator=g3) * 0.02)
            la3 = (torch.randn(r3, k3, device=dev, generator=g3) * 0.01).bfloat16() if r3 else None
            lb3 = (torch.randn(n3, r3, device=dev, generator=g3) * 0.01).bfloat16() if r3 else None
            x3 = torch.randn(m3, k3, device=dev, generator=g3).bfloat16()
            ref3 = linear_forward(x3, full3, k3, n3, _lib.LAYOUT_OUT_IN, lora_a=la3, lora_b=lb3, lora_scale=2.0)
            lin3 = ShardedNf4Linear.from_full(full3, k3, n3, world, rank, lora_a=la3, lora_b=lb3, lora_scale=2.0)
            pp = lin3.peer_store_plan(x3, signal=True)
            for _rep in range(2):
                pp.y.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                pp.run()
                pp.wait(world)
                torch.cuda.synchronize()
                if m3 <= 16:
                    good = torch.equal(pp.y, ref3)
                else:
                    tol = ref3.float().abs() * 2.0 ** -7 + 4e-6 * float(ref3.float().abs().max())
                    good = bool(((pp.y.float() - ref3.float()).abs() <= tol).all())
                good = good and int(pp.arrivals[0].item()) == 0
                if not good:
                    print(f"rank {rank} peer_store_plan case {case}: output differs or counter not back at zero", flush=True)
                ok &= good
                dist.barrier()
            del pp
        d0, d1, d2 = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        ok &= L.nf4_device_status(ctypes.byref(d0), ctypes.byref(d1), ctypes.byref(d2)) == 0
    finally:
        results[rank] = 1 if ok else 0
        torch.cuda.synchronize()
        dist.barrier()
        del peers_y, peers_c, peers_z
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_scattered_decode_forward_on_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Array("i", [0] * world)
    port = _free_port()
    procs = [ctx.Process(target=_scatter_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1] * world


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_forward_on_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Array("i", [0] * world)
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(results) == [1] * world
