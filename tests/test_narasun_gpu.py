"""The Narasun decoder in the engine against the plain implementation (plain_narasun.py): every mechanism in
a model of its own, whole prompts, prompts against token-by-token decoding, portions down to two tokens,
unequal batches against each request alone, slots and pages that are used again, decoding across page and
chunk borders, the first tokens, other sizes (unequal head sizes, one head, several experts per token), and
greedy generation through the library's own entry point."""
import pytest
import torch

import plain_narasun as plain
import tiny_narasun as tiny

pytestmark = pytest.mark.gpu

TOL_F32 = 3e-5            # largest |engine - plain| relative to the largest |logit|: float32 sums against float64
# bfloat16: a row's error relative to the row's largest logit.  The yardstick is the plain implementation with
# roundings to bfloat16 where an engine stores activations: its distance from the exact result is what the storage
# format alone costs on this input (0.005 to 0.03 for the typical row of these models, more in a matrix memory's
# first rows, whose normaliser is small).  A router whose two best scores are closer than that rounding may pick
# the other expert for a token, in either implementation, so single rows may be far off in both: the engine's
# typical row must be as close as the yardstick's (twice its median), and few rows may be far beyond its 90th percentile.
BF16_FACTOR, BF16_SLACK, BF16_ROWS_OVER = 2.0, 0.004, 0.15


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("narasun")
    return {name: tiny.make_folder(tmp, name, seed=10 + i) for i, name in enumerate(tiny.ALL)}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: tiny.load_plain(f) for name, f in folders.items()}


_models = {}


def model_for(folders, name, dtype, **kw):
    from catena_models_b200.api import Model

    key = (name, dtype, tuple(sorted(kw.items())))
    if key not in _models:
        _models[key] = Model.load(folders[name], dtype=dtype, max_tokens=4096, **kw)
    return _models[key]


def row_errs(got, ref):
    ref = ref.to(torch.float64).cpu()
    return (got.to(torch.float64).cpu() - ref).abs().amax(-1) / ref.abs().amax(-1)


def check(got, ref, dtype):
    """ref: the exact logits, or (exact, the yardstick's) for bfloat16."""
    same = None
    if isinstance(ref, tuple):
        ref, same = ref
    assert got.shape == ref.shape
    assert bool(torch.isfinite(got).all())
    errs = row_errs(got, ref)
    if dtype == "float32":
        assert float(errs.max()) < TOL_F32, float(errs.max())
    else:
        yard = row_errs(same, ref)
        assert float(errs.median()) < BF16_FACTOR * float(yard.median()) + BF16_SLACK, (float(errs.median()), float(yard.median()))
        far = 3.0 * float(torch.quantile(yard, 0.9)) + 4 * BF16_SLACK
        assert float((errs > far).double().mean()) <= BF16_ROWS_OVER, (errs, far)


def exact(plains, name, tokens, dtype="float32", choices=None):
    """The plain implementation's logits; for bfloat16 with the yardstick's beside them, both with the experts
    that the engine chose (`choices`, from run_alone): a router's close call may fall the other way in bfloat16,
    in either implementation, and would then hide what the comparison is about (float32 compares the choice too)."""
    cfg, tensors = plains[name]
    ref = plain.forward(cfg, tensors, tokens, choices=choices)
    if dtype == "bfloat16":
        return ref, plain.forward(cfg, tensors, tokens, bf16=True, choices=choices)
    return ref


def run_alone(engine, tokens, cuts, choices=None):
    """One request through the engine in steps of the given sizes (the rest token by token); every logit.
    choices (a list): receives, per run of a routed feed-forward, the experts chosen for every token."""
    from catena_models_b200 import kernels

    (slot,) = engine.admit(1)
    out, at = [], 0
    route, per_step = kernels.moe_route, []

    def spy(ids, wts, perm, dest, work, h, w_router, tok_seq, top, *a, **k):
        route(ids, wts, perm, dest, work, h, w_router, tok_seq, top, *a, **k)
        if not torch.cuda.is_current_stream_capturing():
            per_step[-1].append(ids.view(-1, top).cpu())

    try:
        if choices is not None:
            kernels.moe_route = spy
        for n in list(cuts) + [1] * len(tokens):
            if at >= len(tokens):
                break
            part = tokens[at:at + n]
            per_step.append([])
            out.append(engine.step([slot], [part], [list(range(len(part)))]).float().cpu())
            per_step[-1] = [ids[:len(part)] for ids in per_step[-1]]
            at += len(part)
        engine.check_errors()
    finally:
        kernels.moe_route = route
        engine.release([slot])
    if choices is not None and per_step and per_step[0]:
        choices.extend(torch.cat([step[c] for step in per_step]) for c in range(len(per_step[0])))
    return torch.cat(out)


def engine_for(folders, name, dtype):
    """The module's engine for a model and dtype.  bfloat16 engines of models with a router run kernel by kernel:
    a replayed recording does not pass through the call that `run_alone` listens to (recorded steps are compared
    in float32, and in bfloat16 on model D, which has no router)."""
    routed = any((l.get("mlp") or {}).get("kind") == "moe" for l in tiny.ALL[name]["layers"])
    return model_for(folders, name, dtype, **({"use_graphs": False} if dtype == "bfloat16" and routed else {})).engine


def compare_alone(engine, plains, name, tokens, cuts, dtype):
    """run_alone against the plain implementation (in bfloat16 with the engine's own choice of experts)."""
    choices = [] if dtype == "bfloat16" else None
    got = run_alone(engine, tokens, cuts, choices)
    check(got, exact(plains, name, tokens, dtype, choices or None), dtype)
    return got


@pytest.mark.parametrize("name", list(tiny.ALL))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(folders, plains, name, dtype):
    """Each mechanism's own model and the mixed ones: prompts of 1, 2 and some dozens of tokens, every position."""
    engine = engine_for(folders, name, dtype)
    vocab = plains[name][0]["vocab"]
    for n, seed in ((1, 1), (2, 2), (37, 3), (131, 4)):
        tokens = tiny.prompt(n, vocab, seed)
        compare_alone(engine, plains, name, tokens, [n], dtype)


@pytest.mark.parametrize("name", ["P", "Q", "R", "D", "O"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_continues_a_prompt(folders, plains, name, dtype):
    """40 tokens in one step, then 50 one by one (across the border of a cache page at 64): the state and
    the cache carry everything the later tokens need."""
    engine = engine_for(folders, name, dtype)
    tokens = tiny.prompt(90, plains[name][0]["vocab"], 5)
    compare_alone(engine, plains, name, tokens, [40], dtype)


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_token_by_token_equals_prompt(folders, name):
    """float32: a prompt in one step and the same tokens one by one give the same logits up to the order of sums."""
    engine = model_for(folders, name, "float32").engine
    tokens = tiny.prompt(70, tiny.ALL[name]["vocab"], 6)
    whole, single = run_alone(engine, tokens, [70]), run_alone(engine, tokens, [])
    assert float(row_errs(single, whole).max()) < TOL_F32


@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions(folders, plains, name, dtype):
    """A prompt in portions of several sizes, down to two tokens, some ending on a page border."""
    engine = engine_for(folders, name, dtype)
    tokens = tiny.prompt(150, plains[name][0]["vocab"], 7)
    for cuts in ([2, 2, 60, 3, 61, 22], [64, 64, 2, 20], [7] * 22, [1, 2, 127, 20]):
        compare_alone(engine, plains, name, tokens, cuts, dtype)


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "float32"), ("R", "float32"), ("D", "bfloat16"),
                                        ("attention_mix", "bfloat16"), ("memory", "bfloat16")])
def test_unequal_batch_against_each_alone(folders, plains, name, dtype):
    """Four requests of unequal lengths start together and decode together; the short ones end early, and
    their slots serve a second batch at once.  Every request must come out as it does alone.  (bfloat16 on the
    models without a router: see `exact`.)"""
    engine = model_for(folders, name, dtype).engine
    vocab = plains[name][0]["vocab"]
    for round_ in range(2):
        lens, tails = [1, 45, 97, 13], [3, 9, 5, 12]
        reqs = [tiny.prompt(n + k, vocab, 20 + 7 * round_ + i) for i, (n, k) in enumerate(zip(lens, tails))]
        slots = engine.admit(len(reqs))
        got = [[] for _ in reqs]
        first = engine.step(slots, [r[:n] for r, n in zip(reqs, lens)], [list(range(n)) for n in lens]).float().cpu()
        at = 0
        for i, n in enumerate(lens):
            got[i].append(first[at:at + n])
            at += n
        live = list(range(len(reqs)))
        step = 0
        while live:
            lg = engine.step([slots[i] for i in live], [[reqs[i][lens[i] + step]] for i in live]).float().cpu()
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
            step += 1
            for i in [i for i in live if step >= tails[i]]:
                engine.release([slots[i]])
                live.remove(i)
        engine.check_errors()
        for i, r in enumerate(reqs):
            mine = torch.cat(got[i])
            check(mine, exact(plains, name, r, dtype), dtype)
            if dtype == "float32":
                assert float(row_errs(mine, run_alone(engine, r, [lens[i]])).max()) < TOL_F32


@pytest.mark.parametrize("name", ["P", "Q"])
def test_slots_and_pages_are_used_again(folders, plains, name):
    """A long request leaves its slot; the next request on that slot starts from an empty state and clean pages."""
    from catena_models_b200.api import Model

    model = Model.load(folders[name], dtype="float32", max_tokens=256, max_seqs=1)      # one slot, four pages
    engine = model.engine
    vocab = plains[name][0]["vocab"]
    for n, seed in ((200, 30), (9, 31), (130, 32), (2, 33)):
        tokens = tiny.prompt(n, vocab, seed)
        check(run_alone(engine, tokens, [n // 2]), exact(plains, name, tokens), "float32")
    assert engine.cache.book.slots.free_count == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, plains, dtype):
    """Decoding from 200 to 330 tokens: past the 256 entries of one decode-attention chunk and across three page
    borders, with the query temperature changing every few tokens."""
    name = "Q"
    engine = engine_for(folders, name, dtype)
    tokens = tiny.prompt(330, plains[name][0]["vocab"], 40)
    compare_alone(engine, plains, name, tokens, [200], dtype)


def test_a_far_key_and_a_sink_show(folders, plains):
    """Weights made so that the faults this design invites would show: the first layer's attention gets one
    head whose sink outweighs every score and another whose sink is far below them, and scores large enough for
    single far keys to carry a query's whole weight."""
    from catena_models_b200.api import Model

    name = "attention_mix"
    cfg, tensors = plains[name]
    tensors = dict(tensors)
    tensors["l0.mix.left.sink"] = torch.tensor([6.0, -30.0], dtype=torch.bfloat16)
    tensors["l0.mix.left.q"] = tensors["l0.mix.left.q"] * 6.0
    model = Model(__import__("catena_models_b200.engine.model", fromlist=["DecoderModel"]).DecoderModel.from_tensors(
        cfg, tensors, torch.float32, "cuda:0"), max_tokens=2048)
    tokens = tiny.prompt(600, cfg["vocab"], 50)
    ref = plain.forward(cfg, tensors, tokens)
    check(run_alone(model.engine, tokens, [560]), ref, "float32")
    # and the sink matters: without it the logits are others
    no_sink = dict(tensors)
    no_sink["l0.mix.left.sink"] = torch.tensor([-30.0, -30.0], dtype=torch.bfloat16)
    assert float(row_errs(plain.forward(cfg, no_sink, tokens), ref).max()) > 1e-3


@pytest.mark.parametrize("head", [64, 128])
def test_long_prompts_on_the_tensor_core_attention(tmp_path, head):
    """Heads of 64 and 128 and prompts beyond 768 tokens take the tcgen05 attention kernel in bfloat16: the sink,
    the query temperature (a step every 256 tokens) and a second, shorter prompt in the same step."""
    from catena_models_b200.api import Model

    cfg = dict(architecture="Narasun", vocab=80, width=128, norm=dict(eps=1e-6), loop=None, layers=[
        tiny.parallel(tiny.attention(2, 1, head, head, head ** -0.5, 0.5, 256), 1, 16, 4, 1.0, 0.3, None)])
    folder = tiny.make_folder(tmp_path, f"tc{head}", seed=60 + head, config=cfg)
    pc, pt = tiny.load_plain(folder)
    engine = Model.load(folder, dtype="bfloat16", max_tokens=4096).engine
    a, b = tiny.prompt(1100, 80, 61), tiny.prompt(300, 80, 62)
    slots = engine.admit(2)
    want = [list(range(0, 1100, 7)) + [1099], list(range(0, 300, 5))]
    got = engine.step(slots, [a, b], want).float().cpu()
    nxt = engine.step(slots, [[5], [6]]).float().cpu()
    engine.check_errors()
    engine.release(slots)
    ra, rb = plain.forward(pc, pt, a + [5]), plain.forward(pc, pt, b + [6])
    ya, yb = plain.forward(pc, pt, a + [5], bf16=True), plain.forward(pc, pt, b + [6], bf16=True)
    check(got, (torch.cat([ra[want[0]], rb[want[1]]]), torch.cat([ya[want[0]], yb[want[1]]])), "bfloat16")
    check(nxt, (torch.stack([ra[-1], rb[-1]]), torch.stack([ya[-1], yb[-1]])), "bfloat16")


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation(folders, plains, name):
    """`Model.generate` (scheduler, batches, on-device argmax, recorded decode steps) against the plain greedy loop."""
    model = model_for(folders, name, "float32")
    cfg, tensors = plains[name]
    prompts = [tiny.prompt(n, cfg["vocab"], 70 + n) for n in (5, 23, 1)]
    out = model.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=())
    for p, g in zip(prompts, out):
        assert g.tokens == plain.greedy(cfg, tensors, p, 12)


def test_graphs_and_kernel_by_kernel_agree(folders):
    """Recorded decode steps replay what the kernel-by-kernel step computes."""
    name = "P"
    a = model_for(folders, name, "float32").engine
    b = model_for(folders, name, "float32", use_graphs=False).engine
    tokens = tiny.prompt(40, tiny.ALL[name]["vocab"], 80)
    assert float(row_errs(run_alone(a, tokens, [20]), run_alone(b, tokens, [20])).max()) < 1e-6


def test_checkpoint_copies_every_state(folders, plains):
    """A session set aside and resumed twice: the copies go on from the same keys, values and matrix states."""
    name = "Q"
    model = model_for(folders, name, "float32")
    cfg, tensors = plains[name]
    tokens = tiny.prompt(80, cfg["vocab"], 90)
    s = model.session(capacity=128)
    s.prefill_logits(tokens[:70])
    ckpt = s.into_checkpoint()
    ref = plain.forward(cfg, tensors, tokens)[-1]
    for _ in range(2):
        with model.resume_checkpoint(ckpt) as r:
            got = r.append_logits(tokens[70:])
            assert float(row_errs(got[None], ref[None]).max()) < TOL_F32
    ckpt.close()
