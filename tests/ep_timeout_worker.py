"""Worker of tests/test_gpu_ep_timeout.py (torchrun, one rank per GPU, gloo for the host side).

Both ranks run one expert-parallel forward.  Then rank 1 stays out of the next one (between steps:
nothing of its own is in flight) and rank 0 calls it alone.  Rank 0's collectives cannot complete, so
its bounded host wait must run out (ATENIA_MOE_EP_TIMEOUT_S), abort the communicator and return
ATENIA_ERR_NCCL; afterwards the layer reports ATENIA_ERR_STATE instead of hanging.  No GPU fault is
involved: the waiting NCCL kernel is ended by ncclCommAbort.  With layout "flags" (direct exchange,
ATENIA_MOE_EP_FLAGS=1) there is no collective: rank 0's kernels poll flags that rank 1 never sets, the
bounded poll runs out (ATENIA_MOE_EP_FLAG_TIMEOUT_MS), the forward reports ATENIA_ERR_DEVICE_TIMEOUT and
the next one ATENIA_ERR_STATE; the kernels return normally and the context stays usable."""
import ctypes as C
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main():
    wd = threading.Timer(150.0, lambda: os._exit(4))  # never wait for ever
    wd.daemon = True
    wd.start()
    from ateniaengine_b200 import _lib, synth
    from ateniaengine_b200._lib import AteniaError

    layout = sys.argv[1]  # sharded | replicated | flags (direct exchange synchronised by flags in peer memory)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo")
    shape = synth.small(synth.SHAPES["mixtral"], d_model=256, d_ff=256)
    el = shape.num_experts // world
    w = synth.make_weights(shape, 4, dev, experts=(rank * el, el))
    x = synth.make_activations(shape, 40 + (0 if layout == "replicated" else rank), dev, tokens=32)
    layer = synth.build_layer(shape, w, max_tokens=32, ep_rank=rank, ep_world=world)
    nb = _lib.lib().atenia_moe_ep_unique_id_bytes()
    idt = torch.zeros(nb, dtype=torch.uint8)
    if rank == 0:
        buf = C.create_string_buffer(nb)
        _lib.check(_lib.lib().atenia_moe_ep_get_unique_id(buf), "ep_get_unique_id")
        idt = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
    dist.broadcast(idt, 0)
    layer.ep_init(bytes(idt.numpy().tobytes()))
    if layout == "replicated":
        layer.ep_replicated_tokens(True)
    if layout == "flags":
        mine = torch.frombuffer(bytearray(layer.ep_ipc_export()), dtype=torch.uint8).clone()
        blobs = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(blobs, mine)
        layer.ep_ipc_import(b"".join(bytes(b.numpy().tobytes()) for b in blobs))
    out = layer.forward(x, out_dtype=torch.float32, sync=True)  # a healthy step on both ranks
    assert torch.isfinite(out).all()
    dist.barrier()
    ok = True
    if rank == 0:
        t0 = time.perf_counter()
        status = 0
        try:
            layer.forward(x, out_dtype=torch.float32, sync=True)  # the peer never joins this one
        except AteniaError as e:
            status = e.status
        waited = time.perf_counter() - t0
        after = 0
        try:
            layer.forward(x, out_dtype=torch.float32, sync=True)
        except AteniaError as e:
            after = e.status
        # (with flags the wait that runs out is a kernel's bounded poll: ATENIA_ERR_DEVICE_TIMEOUT)
        ok = status == (-8 if layout == "flags" else -10) and after == -4 and waited < 60.0
        print(f"{layout}: status={status} after={after} waited={waited:.1f}s ok={ok}", flush=True)
    dist.barrier()  # rank 1 has waited here, idle, all along
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
