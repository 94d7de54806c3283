"""The decoder drivers on the CPU.  With the oracle standing in for the device operators
(tests/cpu_context.py), the one-rank driver must give the tokens of the straight-line CPU
decoder, and the tensor-parallel driver -- two and four gloo ranks, every matmul split by rows,
attention on the rank's own heads, four all-gathers per layer, the greedy token picked from the
ranks' best rows -- must give the same tokens on every rank: the row split is exact, so the
sharded decoder is the one-rank decoder bit for bit."""
import json
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
from cpu_context import OracleContext
from __graft_entry__ import load_package

pkg = load_package()
dec = pkg.decoder

LAYERS, HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, VOCAB = 2, 256, 4, 4, 64, 256, 512
PROMPT_LEN, STEPS, SEED = 9, 10, 31


def _model(experts=0):
    cfg = dec.DecoderConfig(LAYERS, HIDDEN, HEADS, KV_HEADS, HEAD_DIM, 128 if experts else INTER,
                            VOCAB, experts=experts, top_k=2 if experts else 0)
    weights = dec.synthetic_weights(cfg, seed=SEED)
    prompt = np.random.default_rng(SEED).integers(0, VOCAB, PROMPT_LEN).tolist()
    return cfg, weights, prompt


def test_one_rank_driver_equals_the_straight_line_decoder():
    cfg, weights, prompt = _model()
    want, _ = ol.dense_decoder_tokens(cfg, weights, prompt, STEPS)
    model = dec.DenseDecoder(OracleContext(), cfg, weights, capacity=PROMPT_LEN + STEPS + 4,
                             device="cpu")
    assert model.generate(prompt, STEPS) == want


def test_one_rank_driver_with_routed_experts():
    cfg = dec.DecoderConfig(2, 256, 4, 2, 64, 128, 512, experts=8, top_k=2)
    weights = dec.synthetic_weights(cfg, seed=4)
    prompt = np.random.default_rng(5).integers(0, 512, 12).tolist()
    want, _ = ol.dense_decoder_tokens(cfg, weights, prompt, 8)
    model = dec.DenseDecoder(OracleContext(), cfg, weights, capacity=32, device="cpu")
    assert model.generate(prompt, 8) == want


def test_layer_shards_reassemble():
    cfg, weights, _ = _model()
    layer, shapes = weights["layers"][0], weights["shapes"]
    world = 4
    parts = [pkg.shard.decoder_layer_shard(cfg, shapes, layer, r, world)[0] for r in range(world)]
    tile = lambda k: (k // 128) * 544
    q_l, kv_l = cfg.q_dim // world, cfg.kv_dim // world
    qs = b"".join(p["qkv"][:(q_l // 8) * tile(HIDDEN)].tobytes() for p in parts)
    ks = b"".join(p["qkv"][(q_l // 8) * tile(HIDDEN):((q_l + kv_l) // 8) * tile(HIDDEN)].tobytes()
                  for p in parts)
    vs = b"".join(p["qkv"][((q_l + kv_l) // 8) * tile(HIDDEN):].tobytes() for p in parts)
    assert qs + ks + vs == layer["qkv"].tobytes()
    assert b"".join(p["o"].tobytes() for p in parts) == layer["o"].tobytes()
    assert b"".join(p["down"].tobytes() for p in parts) == layer["down"].tobytes()
    half = layer["gate_up"].size // 2
    gates = b"".join(p["gate_up"][:p["gate_up"].size // 2].tobytes() for p in parts)
    ups = b"".join(p["gate_up"][p["gate_up"].size // 2:].tobytes() for p in parts)
    assert gates == layer["gate_up"][:half].tobytes() and ups == layer["gate_up"][half:].tobytes()
    with pytest.raises(ValueError):
        pkg.shard.decoder_layer_shard(cfg, shapes, layer, 0, 3)


def _worker(rank, world, port, out_dir, experts):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, weights, prompt = _model(experts)
    model = dec.TensorParallelDecoder(OracleContext(), cfg, weights,
                                      capacity=PROMPT_LEN + STEPS + 4, rank=rank, world=world,
                                      device="cpu")
    tokens = model.generate(prompt, STEPS)
    with open(os.path.join(out_dir, f"tokens_{rank}.json"), "w") as f:
        json.dump(tokens, f)
    dist.destroy_process_group()


@pytest.mark.parametrize("world,experts", [(2, 0), (4, 0), (2, 8), (4, 8)])
def test_tensor_parallel_driver_gives_the_one_rank_tokens(tmp_path, world, experts):
    """experts > 0: attention split by heads, the feed-forward block split by expert with one
    all-reduce of the route rows."""
    cfg, weights, prompt = _model(experts)
    want, margins = ol.dense_decoder_tokens(cfg, weights, prompt, STEPS)
    port = 29500 + (os.getpid() + 7 * world + experts) % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path), experts), nprocs=world, join=True)
    for rank in range(world):
        with open(tmp_path / f"tokens_{rank}.json") as f:
            assert json.load(f) == want, (rank, margins)
