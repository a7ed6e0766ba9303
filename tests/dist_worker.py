"""Child process of the multi-process CPU tests (gloo). Usage: dist_worker.py <scenario> <out_dir>."""

import copy
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from deepfold3_dev_b200.config.schema import TrainingConfig  # noqa: E402
from deepfold3_dev_b200.data.synthetic import batch_features, synthetic_complex  # noqa: E402
from deepfold3_dev_b200.parallel.dist import DistInfo, init_process_group  # noqa: E402
from deepfold3_dev_b200.training.state import TrainState  # noqa: E402
from deepfold3_dev_b200.training.trainer import Trainer  # noqa: E402
from tests.helpers import tiny_config  # noqa: E402


def example(i):
    return synthetic_complex([("protein", 12), ("protein", 8)], num_msa=8, num_templates=0, seed=10 + i)


def make_trainer(info, out_dir, **over):
    mc = tiny_config()
    mc.evoformer.msa_dropout = mc.evoformer.pair_dropout = mc.pairformer.pair_dropout = 0.0
    mc.template.pairformer.pair_dropout = 0.0
    tc = TrainingConfig(diffusion_batch_size=2, dtype="fp32", mini_rollout_steps=1, max_recycles=0, warmup_steps=0,
                        output_dir=out_dir, seed=3, alpha_confidence=0.0, **over)  # fmt: skip
    return Trainer(tc, mc, dist_info=info, device="cpu")


def same_noise_step(trainer, batch):
    """One micro-step with the RNG pinned, so ranks and the single process draw the same diffusion noise."""
    torch.manual_seed(1234)
    trainer.state.global_step = 0
    trainer.micro_step(batch, num_recycles=0)


def main():
    scenario, out_dir = sys.argv[1], sys.argv[2]
    if scenario == "ddp_step":
        info = init_process_group(timeout_s=120, device="cpu")
        tr = make_trainer(info, out_dir)
        same_noise_step(tr, batch_features([example(info.rank)]))
        tr.grad_sync.clip_and_average(tr.optimizer, 0.0, False)
        grad = tr.optimizer.flat_grad.clone()
        tr.engine.add_microstep_loss(torch.zeros(()))
        tr.optimizer.step()
        torch.save({"grad": grad, "params": tr.optimizer.flat_param.clone()}, os.path.join(out_dir, f"rank{info.rank}.pt"))
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    elif scenario == "single_step":
        tr = make_trainer(DistInfo(), out_dir)
        total = None
        for i in range(2):
            tr.optimizer.zero_grad()
            same_noise_step(tr, batch_features([example(i)]))
            total = tr.optimizer.flat_grad.clone() if total is None else total + tr.optimizer.flat_grad
        torch.save({"grad": total / 2}, os.path.join(out_dir, "single.pt"))
    elif scenario == "schedule_free_lockstep":
        # ranks are seeded differently (seed + rank); after the broadcast both sequences (parameters and z) must agree
        info = init_process_group(timeout_s=120, device="cpu")
        tr = make_trainer(info, out_dir, optimizer_type="schedule_free")
        for step in range(2):
            same_noise_step(tr, batch_features([example(info.rank + 2 * step)]))
            tr.engine.step_or_skip(tr.state)
        torch.save({"params": tr.optimizer.flat_param.clone(), "z": tr.optimizer.z.clone()},
                   os.path.join(out_dir, f"sf_rank{info.rank}.pt"))  # fmt: skip
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    elif scenario == "nan_consensus":
        info = init_process_group(timeout_s=60, device="cpu")
        tr = make_trainer(info, out_dir, max_consecutive_nan_skips=0)
        before = tr.optimizer.flat_param.clone()
        same_noise_step(tr, batch_features([example(info.rank)]))
        loss = torch.tensor(float("nan")) if info.rank == 1 else torch.tensor(1.0)
        tr.engine._nan_accum = None
        tr.engine.add_microstep_loss(loss)
        res = tr.engine.step_or_skip(tr.state)
        ok = (not res.advanced) and res.reason == "loss" and res.nan_ranks == [1]
        ok = ok and torch.equal(before, tr.optimizer.flat_param) and tr.state.effective_step == 0
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        sys.exit(0 if ok else 3)
    elif scenario == "stop_file":
        from deepfold3_dev_b200.parallel.dist import ShutdownCoordinator

        stop = os.path.join(out_dir, "STOP")
        os.environ["DF3_STOP_FILE"] = stop
        info = init_process_group(timeout_s=60, device="cpu")
        sc = ShutdownCoordinator(info, install_handlers=False)
        first = sc.tick()
        torch.distributed.barrier()
        if info.rank == 0:
            open(stop, "w").close()
        second = sc.tick()  # only rank 0 sees the file; the MAX all-reduce tells rank 1
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        sys.exit(0 if (not first and second) else 4)
    elif scenario == "peer_exits":
        # rank 1 leaves between steps; rank 0's next collective must fail within the short timeout, not hang
        info = init_process_group(timeout_s=8, device="cpu")
        from deepfold3_dev_b200.parallel.dist import collective_guard

        torch.distributed.barrier()
        if info.rank == 1:
            os._exit(0)
        try:
            with collective_guard("after_peer_exit", info):
                pass
        except RuntimeError as exc:
            sys.exit(0 if "after_peer_exit" in str(exc) else 5)
        sys.exit(6)
    elif scenario == "axial_block":
        from deepfold3_dev_b200.models.evoformer import EvoformerBlock, PairFormerBlock
        from deepfold3_dev_b200.parallel.axial import AxialComm, sharded_trunk
        from tests.helpers import wake_zero_init

        info = init_process_group(timeout_s=120, device="cpu")
        torch.manual_seed(5)
        msa_blocks = torch.nn.ModuleList([EvoformerBlock(16, 32, num_msa_heads=4, num_pair_heads=2, outer_product_hidden=8)]).eval()
        blocks = torch.nn.ModuleList(
            PairFormerBlock(32, 48, num_pair_heads=2, num_single_heads=4, single_key_dim=48, single_value_dim=48) for _ in range(2)
        ).eval()
        wake_zero_init(msa_blocks)
        wake_zero_init(blocks)
        B, S, N = 2, 6, 12 if info.world_size <= 4 else 4 * info.world_size
        pair, single, msa = torch.randn(B, N, N, 32), torch.randn(B, N, 48), torch.randn(B, S, N, 16)
        seq_mask = torch.ones(B, N)
        seq_mask[1, -2:] = 0
        pair_mask = seq_mask[:, :, None] * seq_mask[:, None, :]
        msa_mask = seq_mask[:, None, :].expand(B, S, N).clone()
        msa_mask[0, -1, :3] = 0
        with torch.no_grad():
            want_msa, want_pair, want_single = msa, pair, single
            for blk in msa_blocks:
                want_msa, want_pair = blk(want_msa, want_pair, msa_mask, pair_mask)
            for blk in blocks:
                want_pair, want_single = blk(want_pair, want_single, pair_mask, seq_mask)
        got_msa, got_pair, got_single = sharded_trunk(msa_blocks, blocks, msa, pair, single, msa_mask, pair_mask, seq_mask,
                                                      AxialComm(info, "collective"))  # fmt: skip
        torch.save({"pair_err": (got_pair - want_pair).abs().max(), "single_err": (got_single - want_single).abs().max(),
                    "msa_err": (got_msa - want_msa).abs().max(), "scale": want_pair.abs().max()},
                   os.path.join(out_dir, f"axial_rank{info.rank}.pt"))  # fmt: skip
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    else:
        raise SystemExit(f"unknown scenario {scenario}")


if __name__ == "__main__":
    main()
