"""One rank of the KV-head-sharded decode step with peer stores instead of an all-gather.  Started
by tests/test_peer_outputs_gpu.py under torchrun (one process per GPU):

    every rank builds the same seeded full problem, keeps its slice of the kv-heads (and of the q-heads
    that read them), runs infiniopPagedAttentionMultiOut with its head slice inside every rank's full
    output as destinations, passes the symmetric-memory barrier and compares its full output with the
    whole problem computed locally.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    from datetime import timedelta

    dist.init_process_group("nccl", timeout=timedelta(seconds=90))
    import infinicore_b200 as ib
    from infinicore_b200 import sharding, workloads

    heads, kvh, hd = 32, 8, 128
    full = workloads.build_case("peer_full", dtype=torch.bfloat16, seq_lens=[700, 33, 0, 2048, 1, 129], num_heads=heads, num_kv_heads=kvh,
                                head_size=hd, block_size=16, seed=81).to(dev)
    q_sl, kv_sl = sharding.head_slices(heads, kvh, rank, world)
    q = full.q[:, q_sl].contiguous()
    kc = full.k_cache[:, kv_sl].contiguous()
    vc = full.v_cache[:, kv_sl].contiguous()

    peers = sharding.PeerOutputs(6, heads, hd, torch.bfloat16, dev)
    peers.fill_(4.0)
    torch.cuda.synchronize()
    dist.barrier()  # every rank's buffers are initialised before anyone stores into them
    # Six steps into the two alternating buffers.  The query changes every step (scaled by a power of two, so
    # the expected output is computed locally from the whole problem), and after each barrier the ranks read
    # their full output at different speeds: an odd rank first keeps its stream busy for a while, so an even
    # rank is already storing the next step's rows while the odd one still reads this step's.
    ok, err = True, 0.0
    live = [0, 1, 3, 4, 5]
    busy = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    for step in range(6):
        f = float(2 ** (step % 3 - 1))
        want = ib.paged_attention(full.q * f, full.k_cache, full.v_cache, full.block_tables, full.seq_lens, None, full.scale,
                                  out=torch.full((6, heads, hd), 4.0, dtype=torch.bfloat16, device=dev))
        ib.paged_attention_multi_out(peers.destinations(), q * f, kc, vc, full.block_tables, full.seq_lens, None, full.scale)
        peers.barrier()
        if rank % 2 == 1:
            for _ in range(20):
                busy.fill_(step)
        got = peers.full.clone()
        peers.advance()
        e = (got[live].float() - want[live].float()).abs().max().item()
        err = max(err, e)
        ok = ok and e <= 1e-2 and bool((got[2] == 4.0).all())
    torch.cuda.synchronize()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"PEER_OUTPUTS world={world} max_abs_err={err:.3e} ok={int(flag.item())}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
