"""Rank function of tests/test_convert_tp_lora.py::test_lora_on_every_projection_under_tensor_parallelism (importable by
the spawned ranks): a sharded model with an adapter on all seven projections, prefill + decode steps."""
import torch


def rank_fn(rank, tp_size, unique_id, backend):
    import os
    from zse_b200.cache.cache_manager import KVCacheManager
    from zse_b200.format.loader import ZSELoader
    from zse_b200.lora.manager import LoRAManager
    from zse_b200.models.decoder import DecoderModel
    from zse_b200.parallel.comm import NcclComm
    from zse_b200.parallel.tensor_parallel import TensorParallelGroup
    from zse_b200.runtime.runner import ModelRunner
    g = TensorParallelGroup(tp_size, rank, backend, unique_id)
    loader = ZSELoader(os.environ["ZSE_TEST_MODEL"])
    c = loader.config
    dev = torch.device("cpu")
    model = DecoderModel.from_loader(loader, dev, tp_size=tp_size, rank=rank)
    model.comm = NcclComm(rank, tp_size, dev)
    mgr = LoRAManager(model, dev, max_adapters=2, max_rank=8)
    mgr.load_adapter("all", os.environ["ZSE_TEST_ADAPTER"])
    cache = KVCacheManager(c, dev, block_size=16, num_blocks=16, num_kv_heads=model.plan.num_kv_heads)
    runner = ModelRunner(model, cache, max_batch_seqs=2, max_tokens_per_pass=64, max_seq_len=128)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    slot = mgr.slot_of("all")
    cache.allocate_sequence(1, num_tokens=len(prompt))
    tokens = [int(runner.prefill([(1, prompt, 0)], adapters=[slot])[0])]
    for _ in range(5):
        cache.extend_sequence(1, 1)
        tokens.append(int(runner.decode([1], [tokens[-1]], adapters=[slot])[0]))
    g.destroy()
    return {"tokens": tokens, "a_cols": {m: tuple(mgr._a[(0, m)].shape) for m in ("o_proj", "down_proj", "q_proj")}}
