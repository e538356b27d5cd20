"""Worker of the multi-GPU expert-parallel parity test (launched with torchrun, one rank per GPU).

Every rank routes its own tokens through the expert-parallel layer; rank 0 also runs the same layer
unsharded on the concatenation of all ranks' tokens and compares.  Rows, experts and combine order
are the same in both runs, so the outputs must agree to bf16 rounding noise of the intermediate
buffers (identical here: the same kernels see the same rows) -- the bar is exact equality."""
import ctypes as C
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main():
    import threading
    # a rank whose peer died must not wait for ever
    wd = threading.Timer(200.0, lambda: os._exit(4))
    wd.daemon = True
    wd.start()
    from ateniaengine_b200 import _lib, synth

    name = sys.argv[1]
    T = int(sys.argv[2])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    base = synth.SHAPES[name]
    shape = synth.small(base, d_model=512, d_ff=384, shared_d_ff=256 if base.shared_d_ff else 0)
    el = shape.num_experts // world
    w = synth.make_weights(shape, 4, dev, experts=(rank * el, el))
    Tl = T + 5 * rank
    x = synth.make_activations(shape, 40 + rank, dev, tokens=Tl)
    # one capacity on every rank (the direct exchange requires it)
    layer = synth.build_layer(shape, w, max_tokens=T + 5 * (world - 1), ep_rank=rank, ep_world=world)
    nb = _lib.lib().atenia_moe_ep_unique_id_bytes()
    idt = torch.zeros(nb, dtype=torch.uint8, device=dev)
    if rank == 0:
        buf = C.create_string_buffer(nb)
        _lib.check(_lib.lib().atenia_moe_ep_get_unique_id(buf), "ep_get_unique_id")
        idt = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).to(dev)
    dist.broadcast(idt, 0)
    layer.ep_init(bytes(idt.cpu().numpy().tobytes()))
    if len(sys.argv) > 3 and sys.argv[3] == "direct":
        # direct exchange: rows stored into the owners' buffers over peer mappings
        mine = torch.frombuffer(bytearray(layer.ep_ipc_export()), dtype=torch.uint8).to(dev)
        blobs = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(blobs, mine)
        layer.ep_ipc_import(b"".join(bytes(b.cpu().numpy().tobytes()) for b in blobs))
    outs = []
    for _ in range(2):
        outs.append(layer.forward(x, out_dtype=torch.float32, sync=True))
    assert torch.equal(outs[0], outs[1])
    # a run of forwards with nothing between them (the exchange buffers of one are reused by the next)
    for _ in range(12):
        last = layer.forward(x, out_dtype=torch.float32, sync=False)
    layer.check()
    assert torch.equal(outs[0], last)
    sizes = [T + 5 * r for r in range(world)]
    xs = [torch.empty((n, shape.d_model), dtype=x.dtype, device=dev) for n in sizes]
    ys = [torch.empty((n, shape.d_model), dtype=torch.float32, device=dev) for n in sizes]
    for r in range(world):  # broadcast keeps ragged sizes simple
        if r == rank:
            xs[r].copy_(x)
            ys[r].copy_(outs[0])
        dist.broadcast(xs[r], r)
        dist.broadcast(ys[r], r)
    ok = True
    if rank == 0:
        wf = synth.make_weights(shape, 4, dev)
        full = synth.build_layer(shape, wf, max_tokens=sum(sizes))
        ref = full.forward(torch.cat(xs), out_dtype=torch.float32, sync=True)
        got = torch.cat(ys)
        ok = torch.equal(ref, got)
        print(f"EP{world} {name} tokens={sizes}: equal={ok} max_abs={float((ref - got).abs().max()):.3e}", flush=True)
    dist.barrier()  # peers may still map this rank's buffers until here
    dist.destroy_process_group()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    sys.exit(main())
