"""Expert-parallel layer on GPUs: the CUDA LocalCompute behind EpMoeLayer against
the CPU restatement of Model::moe (src/model/model.cpp:394-466).

World 1 runs on one GPU (pack, plan and the inverse permutation are exercised,
the exchange is elided). World 2 runs as two NCCL ranks when the machine has two
GPUs: experts split contiguously, tokens split by rank, two all-to-all exchanges;
the concatenated outputs must match the single-process CPU result.
Tolerances: 1e-5 relative RMSE while the received rows per expert stay on the
f32-accurate GEMV-class kernels, 1e-3 once the tensor-core grouped GEMMs run."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle_lib as ol
from kanjoos_b200 import synth

pytestmark = pytest.mark.gpu

E, H, F, K = 8, 512, 256, 2
TOL_F32, TOL_TC = 1e-5, 1e-3


def problem(cfg, T):
    bank = synth.expert_bank(cfg, n_experts=E, hidden=H, ffn=F)
    wr, _ = synth.router_weight(cfg, n_experts=E, hidden=H)
    hx = synth.hidden_rows(cfg, T, H)
    return bank, wr, hx


def _layer(bank_np, wr, lo, hi, tc_rows, exchange="gather"):
    from kanjoos_b200 import ep
    from kanjoos_b200.moe import ExpertBank
    local = {k: np.ascontiguousarray(v[lo:hi]) for k, v in bank_np.items()}
    bk = ExpertBank.from_numpy(local, wr)
    cp = ep.CudaCompute(bk.router, K, None, tc_rows_per_expert=tc_rows)
    return ep.EpMoeLayer(bk, E, cp, None, K, exchange=exchange)


@pytest.mark.parametrize("exchange", ["gather", "dispatch"])
@pytest.mark.parametrize("T,tc_rows,tol", [(12, 1 << 30, TOL_F32), (160, 1, TOL_TC)])
def test_world_one_on_gpu(T, tc_rows, tol, exchange):
    from gpu_util import report
    bank, wr, hx = problem(401, T)
    want, _, _ = ol.moe(wr, bank, hx, K)
    layer = _layer(bank, wr, 0, E, tc_rows, exchange)
    got = layer.forward(torch.from_numpy(hx).cuda()).cpu().numpy()
    st = report(got, want, f"expert-parallel layer ({exchange}), world 1, T={T}")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= tol
    if exchange == "dispatch":
        assert layer.last_stats["rows_received"] == T * K


def _rank_main(rank, world, port, out_dir, T, tc_rows, exchange, bf16=False, repeats=1):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        bank, wr, hx = problem(402, T)
        e_loc, t_loc = E // world, T // world
        layer = _layer(bank, wr, rank * e_loc, (rank + 1) * e_loc, tc_rows, exchange)
        x = torch.from_numpy(hx[rank * t_loc:(rank + 1) * t_loc].copy()).cuda()
        if bf16:
            x = x.to(torch.bfloat16)
        for _ in range(repeats):  # repeated steps reuse the exchange buffers
            out = layer.forward(x)
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"out{rank}.npy"), out.cpu().numpy())
        np.save(os.path.join(out_dir, f"rows{rank}.npy"), np.array([layer.last_stats.get("rows_received", -1)]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("exchange", ["gather", "dispatch", "peer"])
@pytest.mark.parametrize("T,tc_rows,tol", [(12, 1 << 30, TOL_F32), (320, 1, TOL_TC)])
def test_two_ranks_match_single_process(tmp_path, T, tc_rows, tol, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from gpu_util import report
    world = 2
    bank, wr, hx = problem(402, T)
    want, chosen, _ = ol.moe(wr, bank, hx, K)
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path), T, tc_rows, exchange), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    st = report(got, want, f"expert-parallel layer ({exchange}), 2 NCCL ranks, T={T}")
    assert st["rel_rmse"] <= tol
    if exchange == "dispatch":
        rows = [int(np.load(tmp_path / f"rows{r}.npy")[0]) for r in range(world)]
        owner_rows = np.bincount(chosen.ravel() // (E // world), minlength=world)
        assert rows == owner_rows.tolist() and sum(rows) == T * K


def test_two_ranks_peer_exchange_fp16_rows_repeated(tmp_path):
    """bf16 rows converted to fp16 before they are published, three steps over the same exchange buffers."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from gpu_util import report
    world, T = 2, 320
    bank, wr, hx = problem(402, T)
    hx = synth.bf16_round(hx)
    want, _, _ = ol.moe(wr, bank, hx, K)
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path), T, 1, "peer", True, 3), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    st = report(got, want, "expert-parallel layer (peer exchange, fp16 rows, 3 steps), 2 NCCL ranks")
    assert st["rel_rmse"] <= TOL_TC


FLAG_WORDS, BARRIER_SLOT, FAR = 4096, 4096 - 64, 1 << 20


def _preset_flags(flags, r, world):
    """Every word far ahead of any epoch the test reaches, except the words this rank writes itself."""
    flags.fill_(FAR)
    flags[r:BARRIER_SLOT:world] = 0
    flags[BARRIER_SLOT + r] = 0


def _emulated_ranks(world, T, cfg=403, n_chunks=1):
    """`world` layer objects inside one process on one GPU: every rank's exchange buffers are ordinary device
    tensors, so a "peer" store is a local store. In each rank's flag words the peers' arrivals are preset far ahead
    of the epochs the test reaches and the rank's arrivals at the other ranks go to a sink, so no wait depends on
    another rank's launches (only on the rank's own copy stream): the ranks' steps run one after another."""
    from kanjoos_b200 import ep
    from kanjoos_b200.moe import ExpertBank
    bank, wr, hx = problem(cfg, T)
    hx = synth.bf16_round(hx)
    e_loc, t_loc = E // world, T // world
    dev = torch.device("cuda")
    bufs = [dict(x=torch.zeros((T, H), dtype=torch.float16, device=dev), pe=torch.zeros(T * K, dtype=torch.int32, device=dev),
                 pw=torch.zeros(T * K, dtype=torch.float32, device=dev),
                 parts=torch.zeros((world, t_loc, H), dtype=torch.float32, device=dev),
                 flags=torch.zeros((FLAG_WORDS,), dtype=torch.int32, device=dev)) for _ in range(world)]
    for r, b in enumerate(bufs):
        _preset_flags(b["flags"], r, world)
    sink = torch.zeros(FLAG_WORDS, dtype=torch.int32, device=dev)  # where a rank's arrivals at its "peers" go
    ranks = []
    for r in range(world):
        ptrs = [[b[name].data_ptr() for b in bufs] for name in ("x", "pe", "pw", "parts")]
        ptrs.append([bufs[j]["flags"].data_ptr() if j == r else sink.data_ptr() for j in range(world)])
        local = {k: np.ascontiguousarray(v[r * e_loc:(r + 1) * e_loc]) for k, v in bank.items()}
        bk = ExpertBank.from_numpy(local, wr)
        ctx = ep.EpPeerContext.from_pointers(world, r, t_loc, H, F, E, K, ptrs, keep=(bufs, sink), n_chunks=n_chunks)
        x = torch.from_numpy(hx[r * t_loc:(r + 1) * t_loc].copy()).cuda().to(torch.bfloat16)
        ranks.append((ctx, bk, x))
    return bank, wr, hx, ranks, bufs


@pytest.mark.parametrize("sm_stores", [(False, False), (False, True), (True, True), (False, True, True)],
                         ids=["copies", "f32_partials", "stores_both_ways", "default"])
@pytest.mark.parametrize("world,n_chunks", [(2, 1), (4, 1), (2, 2), (2, 4), (4, 2)])
def test_layer_object_emulated_ranks_one_gpu(world, n_chunks, sm_stores):
    """The whole data path of knj_ep_forward_launch (row and table stores into every rank's buffers, plan over
    the rank's experts, grouped GEMMs, partial sums into the owners' buffers, rank-ordered sum) with the ranks
    stepped in turn; a rank's result is complete once every rank has stepped after it published its rows, so the
    second round's outputs are the layer's."""
    from gpu_util import report
    T = 320
    bank, wr, hx, ranks, _ = _emulated_ranks(world, T, n_chunks=n_chunks)
    want, _, _ = ol.moe(wr, bank, hx, K)
    for ctx, _, _ in ranks:
        ctx.set_transport(*sm_stores)
    outs = [None] * world
    for _ in range(2):
        for r, (ctx, bk, x) in enumerate(ranks):
            outs[r] = ctx.forward(x, bk.router, None, bk, False, torch.float32)
    # the first rank's second step summed partial rows the later ranks stored one round earlier: same inputs, same rows
    for ctx, _, _ in ranks:
        ctx.status()
    got = np.concatenate([o.cpu().numpy() for o in outs])
    st = report(got, want, f"layer object, {world} emulated ranks on one GPU, T={T}, {n_chunks} chunks")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_TC
    for ctx, _, _ in ranks:
        ctx.close()


def test_layer_object_barrier_gives_up_and_recovers():
    """A rank barrier whose peer never arrives (a flag word that nothing sets) ends at its wait limit with the
    status word raised -- KNJ_E_TIMEOUT on the host -- and the context stays usable: once the peer's word is
    there the next barrier passes and the status is clean."""
    from kanjoos_b200._lib import KnjError
    _, _, _, ranks, bufs = _emulated_ranks(2, 64)
    ctx = ranks[0][0]
    for b in bufs:
        b["flags"].zero_()
    ctx.set_wait(2_000_000)  # about a millisecond
    ctx.barrier()
    with pytest.raises(KnjError) as ei:
        ctx.status()
    assert ei.value.code == -5
    _preset_flags(bufs[0]["flags"], 0, 2)  # the peer's arrivals, far ahead of this rank's epochs
    ctx.set_wait(0)
    bk, x = ranks[0][1], ranks[0][2]
    ctx.forward(x, bk.router, None, bk, False, torch.float32)  # resets the status words, two barriers
    ctx.status()
    for c, _, _ in ranks:
        c.close()
