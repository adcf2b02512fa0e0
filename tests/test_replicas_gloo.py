"""The N > 1 plumbing of the verify path on CPU: two gloo ranks.

The path shards by sequence with no data-path collective; what ranks exchange
is the barrier, the max/sum reduction of the bench totals and the gather of
per-sequence results. Each rank here runs the CPU oracle as a stand-in for its
GPU replica (this is a test: the product path never falls back to it), so the
check is that the sharded job reproduces the single-process result sequence by
sequence."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import pyoracle as yo
from yuuka_b200 import replicas, synth

N_SEQ, K = 5, 4


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def verify_sequence(model, cfg, seq: int):
    """One chain verify step of sequence `seq` on the CPU oracle: (accepted, emitted tokens)."""
    V = cfg["vocab"]
    prompt = synth.uniform_i32(16 + seq, 0, V, 300 + seq)
    st = yo.State(model, 64, yo.KV_F32)
    logits = st.forward(prompt)
    pending = yo.argmax(logits)
    # drafts: the greedy continuation with the third token corrupted for odd sequences
    probe = yo.State(model, 64, yo.KV_F32)
    lg = probe.forward(prompt)
    cont = []
    for _ in range(K + 1):
        t = yo.argmax(lg)
        cont.append(t)
        lg = probe.step(t)
    probe.close()
    drafts = cont[1:K + 1]
    if seq % 2:
        drafts[2] = (drafts[2] + 1) % V
    acc, emitted = st.verify_chain(pending, drafts)[:2]
    st.close()
    return int(acc), [int(t) for t in emitted]


def worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = synth.tiny_config()
    model = yo.Model(cfg, synth.make_model(cfg, "q8_0", seed=7, unit_norms=False))
    mine = replicas.sequences_of_rank(N_SEQ, world, rank)
    acc, toks = [], []
    for s in mine:
        a, e = verify_sequence(model, cfg, s)
        acc.append(a)
        toks.append(e)
    dist.barrier()
    totals = replicas.reduce_totals(dist, "cpu", device_ms=10.0 + rank, wall_s=1.0 + 2 * rank,
                                    emitted=float(sum(a + 1 for a in acc)), accepted=float(sum(acc)))
    acc_all, tok_all = replicas.gather_results(dist, acc, toks, world, N_SEQ)
    if rank == 0:
        np.save(os.path.join(out_dir, "acc.npy"), np.array(acc_all))
        np.save(os.path.join(out_dir, "tok.npy"), np.array([t + [-1] * (K + 1 - len(t)) for t in tok_all]))
        np.save(os.path.join(out_dir, "totals.npy"),
                np.array([totals.device_ms, totals.wall_s, totals.emitted, totals.accepted, totals.ranks]))
    dist.barrier()
    dist.destroy_process_group()


def test_sequences_partition():
    for world in (1, 2, 3, 8):
        seen = sorted(s for r in range(world) for s in replicas.sequences_of_rank(11, world, r))
        assert seen == list(range(11))
        for r in range(world):
            assert all(replicas.rank_of_sequence(s, world) == r for s in replicas.sequences_of_rank(11, world, r))
    with pytest.raises(ValueError):
        replicas.sequences_of_rank(4, 2, 2)
    assert replicas.reduce_totals(None, "cpu", 1.0, 2.0, 3.0, 4.0).ranks == 1


def test_two_ranks_reproduce_the_single_process_result(tmp_path):
    world = 2
    mp.spawn(worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    acc = np.load(tmp_path / "acc.npy")
    tok = np.load(tmp_path / "tok.npy")
    totals = np.load(tmp_path / "totals.npy")
    cfg = synth.tiny_config()
    model = yo.Model(cfg, synth.make_model(cfg, "q8_0", seed=7, unit_norms=False))
    for s in range(N_SEQ):
        a, e = verify_sequence(model, cfg, s)
        assert int(acc[s]) == a
        assert tok[s, :a + 1].tolist() == e[:a + 1]
        assert a == (2 if s % 2 else K)
    # max over ranks of the times, sum over ranks of the tokens
    assert totals.tolist() == [11.0, 3.0, float(sum(int(a) + 1 for a in acc)), float(acc.sum()), 2.0]
