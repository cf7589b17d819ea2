"""Worker for the multi-GPU tests (one process per GPU under torch.distributed.run). Prints RESULT lines that the
pytest side parses; every rank leaves only after a final barrier, with no kernel in flight."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


MICRO = 8            # micro-batches per step over all ranks: divisible by every tested world size (1, 2, 4, 8)


def small_spec(world, backend):
    from parameter_golf_b200.spec import family_preset
    s = family_preset("record_11l")
    m = s.model
    m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads, m.mlp_mult, m.vocab_size = 5, 128, 2, 1, 2.0, 256
    m.xsa_last_n, m.rope.dims = 2, 16
    m.bigram.vocab_size, m.bigram.dim = 96, 64
    m.train_seq_len = m.eval_seq_len = 128
    t = s.train
    t.seq_len, t.world_size, t.backend = 128, world, "cuda_distributed" if world > 1 else "cuda_single"
    t.batch_tokens = MICRO * 4 * 128                 # MICRO micro-batches of 4 sequences, whatever the world size
    t.grad_accum_steps = MICRO // world
    t.distributed_optimizer_backend = backend
    t.tied_embed_lr = 0.01
    s.mode = "record"
    s.allow_unsupported_variants = True
    return s


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.models.engine import EngineBackend
    from parameter_golf_b200.ops import native
    out = {}
    if mode == "collectives":
        from parameter_golf_b200.parallel.symm import SymmetricBuffer
        C = native.load()
        n = 1 << 20
        buf = SymmetricBuffer(n * 4)
        sig, val = SymmetricBuffer(4096), SymmetricBuffer(1024)
        x = buf.view(0, (n,), torch.float32)
        torch.manual_seed(rank)
        x.copy_(torch.randn(n, device="cuda"))
        ref = x.clone()
        dist.all_reduce(ref)
        ref /= world
        stats = torch.zeros(4, device="cuda")
        C.comm_barrier(sig.table, rank, world, 0, 1, native.status_word())
        red = torch.empty(n, device="cuda")
        C.comm_reduce_peers(buf.table, world, 0, n, red, 1.0 / world, stats, 1.0 / world, None, 0, None)
        C.comm_scalar_allreduce(val.table, sig.table, rank, world, 0, 32, 1, stats, native.status_word())
        torch.cuda.synchronize()
        native.check_status()
        out["allreduce_err"] = float((red - ref).abs().max())
        out["sumsq_rel"] = float(abs(stats[0] - ref.pow(2).sum()) / ref.pow(2).sum())
        # reduce-scatter in place on my slice, then fan-out copy = two-shot all-reduce
        a, b = n * rank // world, n * (rank + 1) // world
        mine = buf.view(a * 4, (b - a,), torch.float32)
        C.comm_reduce_peers(buf.table, world, a, b - a, mine, 1.0 / world, None, 0.0, None, 0, None)
        C.comm_barrier(sig.table, rank, world, 64, 1, native.status_word())
        C.comm_push_copy(mine, buf.table, world, rank, a)
        C.comm_barrier(sig.table, rank, world, 0, 2, native.status_word())
        torch.cuda.synchronize()
        native.check_status()
        out["twoshot_err"] = float((x - ref).abs().max())
        # the packaged form used by distributed test-time training, odd length, twice in a row
        from parameter_golf_b200.parallel.peer_allreduce import PeerAllReduce
        par = PeerAllReduce(100_003)
        errs = []
        for rep in range(2):
            torch.manual_seed(100 * rep + rank)
            y = torch.randn(100_003 - 7 * rep, device="cuda")
            yr = y.clone()
            dist.all_reduce(yr)
            par.mean_(y)
            torch.cuda.synchronize()
            native.check_status()
            errs.append(float((y - yr / world).abs().max()))
        out["packaged_err"] = max(errs)
        dist.barrier()
        par.close()
        for bb in (buf, sig, val):
            bb.close()
    else:
        backend_name = "sharded_parallel_muon" if mode == "sharded" else "all_reduce_replicated_muon"
        spec = small_spec(world, backend_name)
        params = gpt.init_params(spec.model, 5)
        be = EngineBackend(spec, {k: v.clone() for k, v in params.items()})
        T = be.engine.T
        g = torch.Generator().manual_seed(11)
        steps = 3
        data = torch.randint(0, 256, (steps, MICRO, T + 1), generator=g).to(torch.int16)      # [step, micro-batch, span]
        per = MICRO // world
        losses = []
        for s in range(steps):
            mine = [data[s, rank * per + i].cuda() for i in range(per)]
            losses.append(be.train_step_spans(mine, 1.0, 0.95, qat=(s == 2), staged=True))
        final = be.final_params()
        torch.cuda.synchronize()
        native.check_status()
        # single-GPU reference on rank 0 with both micro-batches accumulated locally
        if rank == 0:
            spec1 = small_spec(1, "all_reduce_replicated_muon")
            spec1.train.grad_accum_steps = MICRO
            ref = EngineBackend(spec1, {k: v.clone() for k, v in params.items()})
            for s in range(steps):
                ref.train_step_spans([data[s, i].cuda() for i in range(MICRO)], 1.0, 0.95, qat=(s == 2), staged=True)
            rp = ref.final_params()
            errs = {}
            for k in final:
                upd = (rp[k] - params[k]).norm().item()
                errs[k] = (final[k] - rp[k]).norm().item() / max(upd, 1e-12)
            out["worst_rel_update_err"] = max(errs.values())
            out["worst_key"] = max(errs, key=errs.get)
        lt = torch.tensor(losses, device="cuda", dtype=torch.float64)
        dist.all_reduce(lt)
        out["mean_losses"] = (lt / world).tolist()
        dist.barrier()
        if be.dist is not None:
            be.dist.close()
    line = f"RESULT {rank} {json.dumps(out)}"
    if os.environ.get("PGB_RESULT_DIR"):                      # a file per rank: lines of several ranks can interleave on a shared stdout
        with open(os.path.join(os.environ["PGB_RESULT_DIR"], f"result_{rank}.txt"), "w") as fh:
            fh.write(line + "\n")
    print(line, flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
