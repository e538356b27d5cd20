"""Worker of the replicated-token expert-parallel test (torchrun, one rank per GPU).

Every rank passes the same batch; each owns E/world experts of every layer.  One layer and a
three-layer pre-norm stack (eager, captured, replayed) must return, on every rank, exactly what
rank 0 computes with unsharded layers."""
import ctypes as C
import os
import sys
import threading

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main():
    wd = threading.Timer(200.0, lambda: os._exit(4))  # a rank whose peer died must not wait for ever
    wd.daemon = True
    wd.start()
    from ateniaengine_b200 import _lib, synth
    from ateniaengine_b200.moe import RealMoeStack

    name, T = sys.argv[1], int(sys.argv[2])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    base = synth.SHAPES[name]
    shape = synth.small(base, d_model=512, d_ff=384, shared_d_ff=256 if base.shared_d_ff else 0)
    el = shape.num_experts // world
    n_layers = 3
    layers = [synth.build_layer(shape, synth.make_weights(shape, 4 + l, dev, experts=(rank * el, el)), max_tokens=T,
                                ep_rank=rank, ep_world=world) for l in range(n_layers)]
    nb = _lib.lib().atenia_moe_ep_unique_id_bytes()
    idt = torch.zeros(nb, dtype=torch.uint8, device=dev)
    if rank == 0:
        buf = C.create_string_buffer(nb)
        _lib.check(_lib.lib().atenia_moe_ep_get_unique_id(buf), "ep_get_unique_id")
        idt = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).to(dev)
    dist.broadcast(idt, 0)
    layers[0].ep_init(bytes(idt.cpu().numpy().tobytes()))
    for l in layers[1:]:
        l.ep_attach(layers[0])
    for l in layers:
        l.ep_replicated_tokens(True)
    x = synth.make_activations(shape, 40, dev, tokens=T, dtype=torch.float32)  # same seed on every rank
    y1 = layers[0].forward(x, out_dtype=torch.float32, sync=True)
    y2 = layers[0].forward(x, out_dtype=torch.float32, sync=True)
    stack = RealMoeStack(layers, residual=2)
    side = torch.cuda.Stream()
    outs = []
    with torch.cuda.stream(side):
        for _ in range(3):  # eager, capture + replay, replay
            outs.append(stack.forward(x, sync=True).clone())
    side.synchronize()
    ok = torch.equal(y1, y2) and torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    # every rank holds the full result: compare all of them with the unsharded run of rank 0
    full = [synth.build_layer(shape, synth.make_weights(shape, 4 + l, dev), max_tokens=T) for l in range(n_layers)]
    ref1 = full[0].forward(x, out_dtype=torch.float32, sync=True)
    ref_stack = RealMoeStack(full, residual=2).forward(x, sync=True)
    ok = ok and torch.equal(ref1, y1) and torch.equal(ref_stack, outs[0])
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok = bool(flag.item())
    if rank == 0:
        print(f"EP{world} replicated {name} tokens={T}: equal={ok} "
              f"max_abs_layer={float((ref1 - y1).abs().max()):.3e} max_abs_stack={float((ref_stack - outs[0]).abs().max()):.3e}",
              flush=True)
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    sys.exit(main())
