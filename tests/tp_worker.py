"""One rank of the tensor-parallel decoder check (launched by torchrun from
test_gpu_tp.py): every rank builds the same full-model weights, keeps its shard,
wires the peer exchange, decodes greedily and compares with the oracle on rank 0's
CPU.  Prints 'TP_OK' on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import cases  # noqa: E402
import oracle  # noqa: E402

CFG = dict(hidden=512, layers=2, n_q=8, n_kv=2, hd=64, ff=1024, vocab=320, eps=1e-6, rope_base=1e6)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from cpp_tensorlib_b200 import check, lib
    from cpp_tensorlib_b200.decoder import Q4Decoder
    check(lib().tlb_init(local))
    wts = cases.decoder_weights(CFG, 55)
    d = Q4Decoder(CFG, 64, rank, world)
    d.load(wts)
    d.connect()
    d.set_pos(0)
    d.capture()
    port = oracle.load_port()
    o = oracle.PortDecoder(port, CFG, 64)
    o.set_embed(wts["embed"]); o.set_vector(0, 5, wts["onorm"]); o.set_linear(0, 4, port.to_q4(wts["lm_head"]))
    for l, L in enumerate(wts["layers"]):
        for k, i in cases.LINEAR_IDS.items():
            o.set_linear(l, i, port.to_q4(L[k]))
        for k, i in cases.VECTOR_IDS.items():
            o.set_vector(l, i, L[k])
    tok, ok = 5, True
    v0, v1 = d.plan["vocab"]
    for pos in range(10):
        dist.barrier()
        nxt = d.step(tok)
        want, lg = o.step(tok, pos)
        mine = d.logits().cpu().numpy()
        ok &= bool(np.allclose(mine, lg[v0:v1], rtol=1e-3, atol=1e-3)) and nxt == want
        tok = nxt
    # device-resident feedback over the exchange, then the status word
    d.set_pos(0); d.set_token(5)
    dist.barrier()
    d.run(10)
    ok &= d.last_token() == tok
    st = (__import__("ctypes").c_int * 2)()
    ok &= lib().tlb_device_status(st, 0) == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_OK" if int(flag.item()) else "TP_FAIL", flush=True)
    d.close(); o.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
