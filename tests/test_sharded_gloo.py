"""CPU, two gloo ranks: the multi-GPU harness logic (KV-head sharding, start
barrier, max-over-ranks step time, aggregate throughput) with the CPU oracle
standing in for the device step."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mac_attention_b200 import sharding, synth
from oracle import mac_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["MAC_ORACLE_THREADS"] = "2"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = synth.make_decode_case(batch=2, ctx=400, hq=16, hkv=4, capacity=64, seed=5)
        synth.plant_matches(case, hit_fraction=0.5, seed=2)
        cfg = O.DecodeConfig(max_context=512, semantic_pos_ahead=32)
        sh = sharding.shard_case(case, world, rank)
        dist.barrier()
        res = O.decode_step(sh.q_post, sh.q_pre, sh.k, sh.v, sh.req_to_token, sh.req_ids,
                            sh.past_lens, sh.out_cache_loc, sh.query_cache, sh.attn_cache,
                            sh.lse_cache, cfg)
        # step time = max over ranks; work = sum over ranks (the bench's reduction)
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        units = torch.tensor([float(sh.q_post.shape[1])], dtype=torch.float64)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
        gathered = [torch.zeros_like(res.out.float()) for _ in range(world)]
        dist.all_gather(gathered, res.out.float())
        if rank == 0:
            full = O.decode_step(case.q_post, case.q_pre, case.k, case.v, case.req_to_token,
                                 case.req_ids, case.past_lens, case.out_cache_loc,
                                 case.query_cache, case.attn_cache, case.lse_cache, cfg)
            ret["same"] = bool(torch.equal(sharding.gather_heads(gathered), full.out.float()))
            ret["tmax"] = float(t)
            ret["units"] = float(units)
    finally:
        dist.destroy_process_group()


def test_two_rank_kv_head_sharding_over_gloo():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["same"] is True
    assert ret["tmax"] == 2.0 and ret["units"] == 16.0
