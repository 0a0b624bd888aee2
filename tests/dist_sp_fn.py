"""Rank function of tests/test_convert_tp_lora.py::test_sequence_parallel_prefill_matches_all_reduce (importable by the
spawned ranks): one prefill pass of a sharded model with the all-reduce path and with the sequence-parallel path."""
import torch


def rank_fn(rank, tp_size, unique_id, backend):
    import os
    from zse_b200.cache.cache_manager import KVCacheManager
    from zse_b200.format.loader import ZSELoader
    from zse_b200.models.decoder import DecoderModel
    from zse_b200.parallel.comm import NcclComm
    from zse_b200.parallel.tensor_parallel import TensorParallelGroup
    from zse_b200.runtime.runner import ModelRunner
    g = TensorParallelGroup(tp_size, rank, backend, unique_id)            # brings the process group up
    loader = ZSELoader(os.environ["ZSE_TEST_MODEL"])
    c = loader.config
    dev = torch.device("cpu")
    out = {}
    prompt = [(7 * i + 3) % c.vocab_size for i in range(37)]              # 37 rows: not a multiple of the ranks
    for name, sp in (("all_reduce", False), ("sequence_parallel", True)):
        comm = NcclComm(rank, tp_size, dev, sequence_parallel=sp)
        comm.sp_min_rows = 8
        model = DecoderModel.from_loader(loader, dev, tp_size=tp_size, rank=rank)
        model.comm = comm
        cache = KVCacheManager(c, dev, block_size=16, num_blocks=16, num_kv_heads=model.plan.num_kv_heads)
        runner = ModelRunner(model, cache, max_batch_seqs=2, max_tokens_per_pass=64, max_seq_len=128)
        cache.allocate_sequence(1, num_tokens=len(prompt))
        first = runner.prefill([(1, prompt, 0)])
        hidden = model.hidden_rows(runner.buf, len(prompt)).float().clone()
        cache.extend_sequence(1, 1)
        second = runner.decode([1], [int(first[0])])                      # one row: below the threshold, all-reduce
        out[name] = {"tokens": [int(first[0]), int(second[0])], "hidden": hidden, "sp_passes": comm.sp_passes}
    g.destroy()
    a, b = out["all_reduce"], out["sequence_parallel"]
    return {"tokens_equal": a["tokens"] == b["tokens"], "tokens": b["tokens"],
            "max_diff": float((a["hidden"] - b["hidden"]).abs().max()),
            "scale": float(a["hidden"].abs().max()), "sp_passes": (a["sp_passes"], b["sp_passes"])}
