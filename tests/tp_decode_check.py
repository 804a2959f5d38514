"""Tensor-parallel greedy decoding against the CPU oracle; run one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 tests/tp_decode_check.py

Every rank loads its shares of the same synthetic model, the group decodes 64 tokens, and rank 0
compares them with the oracle's single-device tokens.  Exits non-zero on a mismatch.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> int:
    import faulthandler

    faulthandler.dump_traceback_later(int(os.environ.get("TP_CHECK_LIMIT", "240")), exit=True)  # a stuck rank says where
    import torch
    import torch.distributed as dist

    import neura_b200 as nb
    import oracle
    from neura_b200 import parallel, qwen
    from oracle.decoder import OracleDecoder, synthetic_model

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # 8 key heads so that the model splits over 2, 4 and 8 ranks; K shares of 128 and 352 straddle super-blocks at 8
    config = qwen.Config("tiny-tp-q4_k", 2, 1024, 8, 8, 128, 2816, 2048, nb.Q4K)
    batch = 2
    packed, norms = synthetic_model(config, seed=23)
    prompts = (oracle.Stream(29).uniform(batch * 12, 0.0, 1.0) * config.vocab).astype(np.uint32).reshape(batch, 12)
    rt = nb.Runtime(local)
    rt.use_stream(rt.new_stream())
    device = torch.device("cuda", local)
    shard = parallel.Shard(config, world, rank, attention=os.environ.get("TP_ATTENTION", "split"))
    stream = torch.cuda.ExternalStream(rt.stream.value, device=device)
    if os.environ.get("TP_COMM", "peer") == "peer":   # the library's own all-reduce over NVLink peer memory
        comm = parallel.PeerComm(rt, world, rank, batch * config.hidden, device=device, stream=stream)
    else:                                              # NCCL through torch.distributed
        comm = parallel.TorchComm(world, rank, device=device, stream=stream)
    weights, dnorms = parallel.load_decoder_weights(rt, config, packed, norms, shard)
    decoder = qwen.Decoder(rt, config, weights, dnorms, batch=batch, capacity=96, shard=shard, comm=comm)
    decoder.fold = os.environ.get("TP_FOLD", "0") == "1"   # exchanges in the products' epilogues (the peer transport only)
    eager = decoder.generate(prompts, 64)
    if os.environ.get("TP_STEP", "graph") == "persistent":   # the whole step as one cooperative kernel a rank
        decoder.compile()
    else:
        decoder.record()
    replayed = decoder.generate(prompts, 64)
    status = 0
    if rank == 0:
        want, margins = OracleDecoder(config, packed, norms, batch=batch, capacity=96).generate(prompts, 64)
        if not np.array_equal(eager, replayed):
            at = np.argwhere(eager != replayed)[0]
            print(f"FAIL: the recorded step decodes other tokens than the eager step, first at {tuple(at)}")
            status = 1
        differs = np.argwhere(eager != want)
        if differs.size:
            b, at = differs[0]
            print(f"FAIL: sequence {b} leaves the oracle at step {at}: {eager[b, at]} for {want[b, at]} "
                  f"(oracle margin {margins[b, at]:.3e})")
            status = 1
        how = type(comm).__name__ + (", attention whole on every rank" if shard.whole else "") + \
            (", exchanges folded into the products" if decoder.fold else "") + \
            (", the step as one persistent kernel" if decoder.compiled is not None else "")
        verdict = (f"tp{world}: 64 greedy tokens x {batch} sequences match the oracle, eager and recorded "
                   f"({how})") if status == 0 else f"tp{world}: FAILED ({how})"
        print(verdict)
        # a record of the run for boxes whose test collection has fewer GPUs than this check wants
        log = os.environ.get("TP_CHECK_LOG")
        if log:
            os.makedirs(os.path.dirname(log) or ".", exist_ok=True)
            with open(log, "a") as fh:
                fh.write(verdict + "\n")
    flag = torch.tensor([status], device=device)
    dist.broadcast(flag, 0)
    rt.sync()
    dist.barrier()
    torch.cuda.synchronize()
    code = int(flag.item())
    # a recorded program holds NCCL kernels, and tearing the process group down under it was seen to
    # wait forever: leave without the teardown, the process is ending anyway
    sys.stdout.flush()
    os._exit(code)


if __name__ == "__main__":
    sys.exit(main())
