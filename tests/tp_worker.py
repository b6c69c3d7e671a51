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


def seven_b_case():
    """BASELINE config 5's shape with 2 layers and the full vocabulary, caches pre-filled to 4096
    (TLB_TP_CFG=7b2): the shard plan of the real model -- at 8 ranks 4,3,4,3 query heads per rank
    with every KV head on two ranks."""
    cfg = dict(cases.QWEN7, layers=2)
    rng = np.random.Generator(np.random.Philox(4))
    E, HD, NQ, NKV, FF, V = cfg["hidden"], cfg["hd"], cfg["n_q"], cfg["n_kv"], cfg["ff"], cfg["vocab"]
    f = lambda *shape: rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
    w = {"embed": f(V, E), "onorm": 1 + f(E), "lm_head": f(E, V), "layers": []}
    for _ in range(cfg["layers"]):
        w["layers"].append(dict(wqkv=f(E, (NQ + 2 * NKV) * HD), wo=f(NQ * HD, E), wgu=f(E, 2 * FF), wd=f(FF, E),
                                bq=f(NQ * HD), bk=f(NKV * HD), bv=f(NKV * HD), an=1 + f(E), fn=1 + f(E)))
    kv = [(rng.standard_normal((NKV, 4096, HD), dtype=np.float32), rng.standard_normal((NKV, 4096, HD), dtype=np.float32))
          for _ in range(cfg["layers"])]
    return cfg, w, kv


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from cpp_tensorlib_b200 import check, lib
    from cpp_tensorlib_b200.decoder import Q4Decoder
    check(lib().tlb_init(local))
    big = os.environ.get("TLB_TP_CFG") == "7b2"
    if big:
        CFG_, wts, kv = seven_b_case()
        pos0, max_ctx, steps = 4096, 4200, 6
    else:
        CFG_, wts, kv = CFG, cases.decoder_weights(CFG, 55), None
        pos0, max_ctx, steps = 0, 64, 10
    d = Q4Decoder(CFG_, max_ctx, rank, world)
    d.load(wts)
    d.connect()
    # the oracle runs on rank 0 only (one host copy of the model); its logits and token are
    # broadcast to the other ranks, which check their own vocabulary shard
    o = None
    if rank == 0:
        port = oracle.load_port()
        o = oracle.PortDecoder(port, CFG_, max_ctx)
    if kv:
        for l, (K, V) in enumerate(kv):
            d.fill_kv(l, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
            if o:
                o.fill_kv(l, K, V)
    d.set_pos(pos0)
    d.capture()
    if o:
        o.set_embed(wts["embed"]); o.set_vector(0, 5, wts["onorm"]); o.set_linear(0, 4, port.to_q4(wts["lm_head"]))
        for l, L in enumerate(wts["layers"]):
            for k, i in cases.LINEAR_IDS.items():
                o.set_linear(l, i, port.to_q4(L[k]))
            for k, i in cases.VECTOR_IDS.items():
                o.set_vector(l, i, L[k])
    tok, ok = 5, True
    v0, v1 = d.plan["vocab"]
    for pos in range(pos0, pos0 + steps):
        dist.barrier()
        nxt = d.step(tok)
        ref = torch.empty(CFG_["vocab"] + 1, device="cuda")
        if o:
            want, lg = o.step(tok, pos)
            ref[:-1] = torch.from_numpy(lg).cuda()
            ref[-1] = float(want)
        dist.broadcast(ref, 0)
        lg, want = ref[:-1].cpu().numpy(), int(ref[-1].item())
        mine = d.logits().cpu().numpy()
        ok &= bool(np.allclose(mine, lg[v0:v1], rtol=1e-3, atol=1e-3)) and nxt == want
        tok = nxt
    # device-resident feedback over the exchange, then the status word
    d.set_pos(pos0); d.set_token(5)
    dist.barrier()
    d.run(steps)
    ok &= d.last_token() == tok
    st = (__import__("ctypes").c_int * 2)()
    ok &= lib().tlb_device_status(st, 0) == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_OK" if int(flag.item()) else "TP_FAIL", flush=True)
    d.close()
    if o:
        o.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
