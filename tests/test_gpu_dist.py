"""Two ranks on two GPUs over NCCL: token shards -> Hessian reduce to owners -> solve -> broadcast,
through the public oneshot() / GPTQModifier path.  Skipped on a single-GPU box."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, scheme, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world,
                                         device_id=torch.device("cuda", rank))
    try:
        here = os.path.dirname(os.path.abspath(__file__))
        for path in (here, os.path.dirname(here)):
            if path not in sys.path:
                sys.path.insert(0, path)
        import test_gpu_oneshot as t
        from llm_compressor_b200 import GPTQModifier, oneshot

        t.DEV = f"cuda:{rank}"
        model = t.tiny_llama()
        recipe = GPTQModifier(targets="Linear", scheme=scheme, ignore=["lm_head"], actorder=None)
        model = oneshot(model, recipe=recipe, dataset=t.calib(), num_calibration_samples=16)
        out = {n: p.data.float().cpu() for n, p in model.named_parameters() if n.endswith("proj.weight")}
        q.put((rank, out, dict(recipe.losses)))
    finally:
        torch.distributed.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("scheme", ["W4A16"])
def test_two_rank_gptq_equals_single_rank(scheme):
    import test_gpu_oneshot as t
    from llm_compressor_b200 import GPTQModifier, oneshot

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, scheme, q)) for r in range(2)]
    for p in procs:
        p.start()
    outs = sorted([q.get(timeout=180) for _ in procs], key=lambda o: o[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, w0, l0), (_, w1, l1) = outs
    # every rank ends with the same weights (owners broadcast their results)
    assert set(w0) == set(w1) and len(w0) == 14
    for n in w0:
        assert torch.equal(w0[n], w1[n]), n
    # and they agree with the single-process run: the Hessian is summed in another order, so a
    # few codes may flip
    recipe = GPTQModifier(targets="Linear", scheme=scheme, ignore=["lm_head"], actorder=None)
    ref = oneshot(t.tiny_llama(), recipe=recipe, dataset=t.calib(), num_calibration_samples=16)
    ref_w = {n: p.data.float().cpu() for n, p in ref.named_parameters() if n.endswith("proj.weight")}
    for n in ref_w:
        layer0 = ".layers.0." in n
        mism = float((ref_w[n] != w0[n]).float().mean())
        assert mism <= (0.01 if layer0 else 0.2), (n, mism)
    # each module's loss was computed by exactly one rank
    assert set(l0) | set(l1) == set(recipe.losses) and not (set(l0) & set(l1))
