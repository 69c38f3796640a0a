"""The entry point for callers that must not allocate device memory while they run a model (a serving
loop that cannot afford cudaMalloc's device-wide synchronisation, or a host with a fixed device-memory
budget): spnb_execute_device_noalloc keeps the model image and the interpreter's spill scratch in a
32 MiB device array that belongs to the library.  Its results must equal those of the regular
device-pointer entry point, on two calls in a row (the array keeps the first call's contents), and for a
second plan that replaces the first one's image.

This file sorts last on purpose: a failure here cannot mask the other GPU tests in a stop-at-first-failure
run.  It passes alone in a fresh process as well as after the rest of the suite."""
import os

import numpy as np
import pytest

from tests.util_models import REL_TOL_F32, max_rel_err, oracle_eval, small_configs, write_query

pytestmark = pytest.mark.gpu


def _both_entries(capi, plan, x, warm=False):
    import torch
    n = x.shape[0]
    dx = torch.from_numpy(x).cuda()
    ref = torch.empty(n, dtype=torch.float32, device="cuda")
    got = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    plan.execute_device(0, n, dx.data_ptr(), ref.data_ptr(), s)
    plan.execute_device_noalloc(0, n, dx.data_ptr(), got.data_ptr(), s)
    torch.cuda.synchronize()
    if warm:
        # the plan's image is resident now: another call must leave the device's free memory where it is
        # (an allocation would show as 2 MiB or more)
        free_before = torch.cuda.mem_get_info()[0]
        plan.execute_device_noalloc(0, n, dx.data_ptr(), got.data_ptr(), s)
        torch.cuda.synchronize()
        assert free_before - torch.cuda.mem_get_info()[0] < (1 << 20)
    return got.cpu().numpy(), ref.cpu().numpy()


def test_noalloc_entry_matches_regular_entry_twice_in_a_row(tmp_path):
    from spnb import capi
    assert capi.device_count() > 0
    plans = []
    for idx, slots in ((4, 6), (2, 0)):  # the first plan spills most of its values to the scratch area
        name, spn, inputs, log_space, marginal = small_configs()[idx]
        q = write_query(spn, marginal, directory=str(tmp_path))
        opts = {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "interp"}
        if slots:
            opts["spnb-interp-slots"] = str(slots)
        plan_path, _ = capi.compile_query(q, opts)
        plans.append((name, q, inputs, capi.Plan(plan_path), plan_path))
    for rounds in range(2):           # second round: each plan's image replaces the other's in the array
        for name, q, inputs, plan, _ in plans:
            for call in range(2):     # two calls in a row share the array and what the first left in it
                x = inputs(50001 + 1000 * call)
                got, ref = _both_entries(capi, plan, x, warm=call == 1)
                assert max_rel_err(got, ref) <= REL_TOL_F32, (name, rounds, call)
                assert max_rel_err(got, oracle_eval(q, x, True)) <= REL_TOL_F32, (name, rounds, call)
    for _, _, _, plan, path in plans:
        plan.close()
        os.remove(path)


def test_noalloc_entry_rejects_what_does_not_fit(tmp_path):
    from spnb import capi
    import torch
    # linear-space plans have no interpreter program
    name, spn, inputs, log_space, marginal = small_configs()[0]
    q = write_query(spn, marginal, directory=str(tmp_path))
    plan_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "false"})
    plan = capi.Plan(plan_path)
    x = torch.from_numpy(inputs(64)).cuda()
    out = torch.empty(64, dtype=torch.float64, device="cuda")
    with pytest.raises(capi.SpnbError, match="log-space"):
        plan.execute_device_noalloc(0, 64, x.data_ptr(), out.data_ptr(), 0)
    plan.close()
    os.remove(plan_path)
    # a model whose op stream alone is larger than the 32 MiB array
    from spnb import synth
    big = synth.config5(repetitions=10)
    q = str(tmp_path / "big.bin")
    with open(q, "wb") as f:
        f.write(big.to_xspn_bytes())
    plan_path, _ = capi.compile_query(q, {"target": "CUDA", "use-log-space": "true", "spnb-kernel": "interp"})
    plan = capi.Plan(plan_path)
    x = torch.from_numpy(synth.config5_inputs(32)).cuda()
    out = torch.empty(32, dtype=torch.float32, device="cuda")
    with pytest.raises(capi.SpnbError, match="32 MiB"):
        plan.execute_device_noalloc(0, 32, x.data_ptr(), out.data_ptr(), 0)
    plan.close()
    os.remove(plan_path)
