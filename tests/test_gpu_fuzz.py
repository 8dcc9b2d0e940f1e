"""Seeded random cases over every kernel family, against the oracle: segment size, element count
(whole segments, often not whole tiles or work units), output type and algorithm are drawn at
random, so that the boundaries between launch shapes are crossed in ways the fixed lists of the
other tests do not spell out."""
import random

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

POW2 = [16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384]
OTHER = [48, 80, 176, 1000, 2040, 24, 3, 100, 4099, 32768, 65536]


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def draw_cases(seed, count):
    rng = random.Random(seed)
    cases = []
    for _ in range(count):
        s = rng.choice(POW2 if rng.random() < 0.7 else OTHER)
        # up to ~2^22 elements; sometimes few segments, sometimes many more than the GPU has SMs x 8
        segs = max(1, int(2 ** rng.uniform(0, 22)) // s)
        if rng.random() < 0.3:
            segs = rng.randint(1, 40)
        op = rng.choice(["reduce", "scan"])
        out32 = rng.random() < 0.5
        algos = ["auto"]
        if s in POW2:
            algos.append("mma")
            if op == "reduce":
                algos.append("shuffle")
                if s <= 2048 and (s * segs) % 64 == 0:
                    algos.append("tcgen05")
            elif (s * segs) % 64 == 0:
                algos.append("tcgen05")
        cases.append((s, segs, op, out32, rng.choice(algos), rng.randrange(1 << 30)))
    return cases


@pytest.mark.parametrize("batch", range(12))
def test_random_cases_match_the_oracle(batch):
    import tcu_scope_b200 as tcu
    for s, segs, op, out32, algo, seed in draw_cases(1000 + batch, 60):
        n = s * segs
        x = tcu.fill(torch.empty((n + 7) // 8 * 8, dtype=torch.float16, device="cuda"), seed, 0)[:n]
        dtype = torch.float32 if out32 else torch.float16
        n_out = segs if op == "reduce" else n
        buf = torch.full((n_out + 128,), -777.0, dtype=dtype, device="cuda")
        out = buf[64:64 + n_out]
        what = (s, segs, op, dtype, algo)
        if op == "reduce":
            tcu.segmented_reduce(x, s, out=out, algo=algo)
            ref = oracle.c_segmented_reduce(bits(x), s)
        else:
            tcu.segmented_scan(x, s, out=out, algo=algo)
            ref = oracle.c_segmented_scan(bits(x), s)
        if out32:
            bad, max_abs, _ = oracle.np_check_f32(out.cpu().numpy(), ref, 1e-3, 1e-5)
            assert bad == 0, (what, max_abs)
        else:
            assert oracle.np_check_f16(bits(out), ref, 2)[0] == 0, what
        guards = torch.cat([buf[:64], buf[64 + n_out:]]).float().cpu()
        assert torch.all(guards == -777.0), what
    assert tcu.device_error() == 0
