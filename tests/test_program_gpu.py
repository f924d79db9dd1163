"""The opt-in decode programs (a decode step as one resident kernel that interprets a list
of operations) against the plain implementation and against the ordinary chain of kernels.
"""
import numpy as np
import pytest
import torch

from conftest import TINY
from test_replay_gpu import TOL, _close, _prompts

pytestmark = pytest.mark.gpu


def _engine(model_dir, programs, max_tokens=512, graphs=True):
    from sandyrt_b200.engine.step import Engine
    from sandyrt_b200.models.model import load_model

    model = load_model(model_dir, device="cuda:0", dtype=torch.bfloat16)
    eng = Engine(model, max_tokens=max_tokens, page_size=16, max_requests=8, use_cuda_graphs=graphs,
                 use_decode_programs=programs)
    eng.cache.device_caches.poison()
    return eng


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("graphs", [False, True])
def test_decode_steps_as_programs(model_dirs, plain_models, name, graphs):
    """Three requests of different lengths: prompts in one step each, then 40 decode steps of all
    three together (one program, recorded once and run again and again; with graphs it is
    captured too).  Every decode step's logits against the plain implementation."""
    from sandyrt_b200.engine.step import StepEntry

    eng = _engine(model_dirs[name], programs=True, graphs=graphs)
    plain = plain_models(name, "bf16")
    n_dec = 40
    seqs = _prompts(name, [7 + n_dec, 33 + n_dec, 70 + n_dec], seed=11)
    want = [plain.logits(ids) for ids in seqs]
    for i, ids in enumerate(seqs):
        eng.step([StepEntry(f"r{i}", ids[:len(ids) - n_dec], [])])
    for j in range(n_dec):
        entries = [StepEntry(f"r{i}", [ids[len(ids) - n_dec + j]], [0]) for i, ids in enumerate(seqs)]
        got = eng.step(entries).cpu().numpy()
        for i, ids in enumerate(seqs):
            _close(got[i:i + 1], want[i][len(ids) - n_dec + j][None], "bfloat16",
                   f"tiny {name}, request {i}, decode step {j} as a program")
    # tiny C has heads of 48, which the interpreter's attention does not take: its steps must
    # have gone through the ordinary kernels (and still be right)
    head = TINY[name]["n_embd"] // TINY[name]["n_head"]
    if head not in (16, 32, 64, 128, 256):
        assert eng.program_runs == 0
    elif graphs:
        # launched once by hand and once under capture; from then on the graph replays the launch
        assert eng.program_runs == 2 and eng.graph_replays == n_dec - 1
    else:
        assert eng.program_runs == n_dec
    eng.check_status()
    eng.cache.alloc.check()


def test_program_matches_the_chain_of_kernels(model_dirs):
    """The same decode steps with and without programs: the two paths round at the same places,
    so their logits agree far inside the bfloat16 tolerance."""
    from sandyrt_b200.engine.step import StepEntry

    outs = []
    for programs in (False, True):
        eng = _engine(model_dirs["B"], programs=programs)
        ids = _prompts("B", [90], seed=5)[0]
        eng.step([StepEntry("r", ids[:50], [])])
        rows = [eng.step([StepEntry("r", [t], [0])]).cpu().numpy().copy() for t in ids[50:]]
        outs.append(np.concatenate(rows))
        assert (eng.program_runs > 0) == programs
    err = np.abs(outs[0] - outs[1]).max()
    assert err < TOL["bfloat16"]["atol"], f"programs and kernels differ by {err}"


def test_program_timeline(model_dirs):
    """The optional timeline: one start mark, then per operation two marks inside it and one after
    its barrier, in order."""
    from sandyrt_b200.engine.step import StepEntry

    eng = _engine(model_dirs["A"], programs=True, graphs=False)
    ids = _prompts("A", [20], seed=2)[0]
    eng.step([StepEntry("r", ids[:10], [])])
    eng.step([StepEntry("r", [ids[10]], [0])])
    (prog, _, _), = [hit for hit in eng._programs.values() if hit is not None]
    n_layers = TINY["A"]["n_layer"]
    assert prog.n_ops == 1 + 5 * n_layers + 2          # embedding, five operations a layer, final norm, head
    tl = torch.zeros(3 * prog.n_ops + 1, dtype=torch.int64, device="cuda:0")
    prog.run(tl)
    torch.cuda.synchronize()
    t = tl.cpu().numpy()
    ends = t[0::3]
    assert (np.diff(ends) > 0).all(), "operations must end one after the other"
    assert 0 < (ends[-1] - ends[0]) < 50_000_000       # nanoseconds
    eng.check_status()


def test_parts_that_cannot_be_recorded_fall_back(model_dirs):
    """float32 engines never use programs; a bfloat16 engine with more tokens in a step than the
    interpreter takes runs that step through the ordinary kernels."""
    from sandyrt_b200.engine.step import Engine, StepEntry
    from sandyrt_b200.models.model import load_model

    model = load_model(model_dirs["A"], device="cuda:0", dtype=torch.float32)
    eng = Engine(model, max_tokens=256, max_requests=8, use_decode_programs=True)
    assert not eng.use_decode_programs
    model = load_model(model_dirs["A"], device="cuda:0", dtype=torch.bfloat16)
    eng = Engine(model, max_tokens=1024, max_requests=32, use_decode_programs=True)
    prompts = _prompts("A", [5] * 20, seed=1)
    for i, ids in enumerate(prompts):
        eng.step([StepEntry(i, ids, [])])
    eng.step([StepEntry(i, [1], [0]) for i in range(20)])      # 20 rows: more than a program takes
    assert eng.program_runs == 0
    eng.step([StepEntry(i, [2], [0]) for i in range(12)])      # 12 rows: a program
    assert eng.program_runs == 1
    eng.check_status()
