"""CPU, world_size 2 over gloo: row-sharded quantization reassembles bit for bit."""
import os
import pathlib
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_row_shards_cover_and_align():
    from nvfp4quant_test_b200.sharding import row_shards, scale_slab

    for rows in (1, 127, 128, 129, 300, 8192, 8192 + 5):
        for world in (1, 2, 3, 4, 8):
            sh = row_shards(rows, world)
            assert len(sh) == world and sh[0][0] == 0 and sh[-1][1] == rows
            for (a, b), (c, d) in zip(sh, sh[1:]):
                assert b == c and a <= b
            assert all(a % 128 == 0 or a == rows for a, _ in sh)
            sizes = [(b - a + 127) // 128 for a, b in sh]
            assert max(sizes) - min(sizes) <= 1
            # scale slabs tile the global buffer without gaps
            end = 0
            for a, b in sh:
                if b > a:
                    lo, hi = scale_slab(a, b, 13)
                    assert lo == end
                    end = hi
            assert end == ((rows + 127) // 128 * 128) * 16
    with pytest.raises(ValueError):
        scale_slab(5, 128, 4)


def _worker(rank, world, port, rows, cols, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cases as C
        from oracle import oracle as O

        from nvfp4quant_test_b200 import sharding as S

        x = C._laplace((rows, cols), 77)
        imp = (C._laplace((64, cols), 78).float() ** 2).sum(0, keepdim=True)
        a, b = S.row_shards(rows, world)[rank]
        x_local = x[a:b].contiguous()
        # global amax over sharded data: 4-byte MAX all-reduce
        local_amax = x_local.float().abs().max() if b > a else torch.tensor(0.0)
        gs, gs_inv = S.global_amax_scale(local_amax, 256.0)
        assert float(gs_inv) == C.global_scale_cpu(x, 256.0)[1]

        def quantize(xl, importance):
            codes, scales = O.quant(1, O.bf16_bits(xl), float(gs_inv), importance.numpy(), lower=-8, upper=7)
            return torch.from_numpy(codes), torch.from_numpy(scales)

        codes, scales, _ = S.quantize_row_shard(quantize, rows, x_local, rank, world, importance=imp)
        full_codes, full_scales = S.gather_rows(codes, scales, rows, cols // 16)
        ref_codes, ref_scales = O.quant(1, O.bf16_bits(x), float(gs_inv), imp.numpy(), lower=-8, upper=7)
        ok = np.array_equal(full_codes.numpy(), ref_codes) and np.array_equal(full_scales.numpy(), ref_scales.reshape(-1))
        pathlib.Path(tmp, f"rank{rank}.ok").write_text("1" if ok else "0")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,cols", [(300, 208), (129, 64)])
def test_sharded_quantization_matches_single_rank(tmp_path, rows, cols):
    world = 2
    port = 29500 + (os.getpid() % 2000) + rows % 7
    mp.spawn(_worker, args=(world, port, rows, cols, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.ok").read_text() == "1"


def _imp_worker(rank, world, port, n, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvfp4quant_test_b200 import sharding as S

        g = torch.Generator().manual_seed(5)
        full = torch.rand(n, generator=g) * 100.0
        scales = torch.tensor([0.25, 0.75, 0.5][:world])
        a, b = S.importance_shards(n, world)[rank]
        imp, gs, gs_inv = S.gather_importance_and_scale(full[a:b].clone(), scales[rank], n)
        ok = (imp.shape == (1, n) and torch.equal(imp.reshape(-1), full) and float(gs) == float(scales.max())
              and float(gs_inv) == float(torch.tensor(1.0) / scales.max()))
        try:
            S.gather_importance_and_scale(full[a:b][:-1], scales[rank], n)
            ok = False
        except ValueError:
            pass
        pathlib.Path(tmp, f"rank{rank}.ok").write_text("1" if ok else "0")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 8192), (3, 208)])
def test_sharded_importance_gathers_to_the_full_vector_and_the_max_scale(tmp_path, world, n):
    from nvfp4quant_test_b200.sharding import importance_shards

    sh = importance_shards(n, world)
    assert sh[0][0] == 0 and sh[-1][1] == n and all(a % 16 == 0 or a == n for a, _ in sh)
    port = 31500 + (os.getpid() % 2000) + world
    mp.spawn(_imp_worker, args=(world, port, n, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.ok").read_text() == "1"
