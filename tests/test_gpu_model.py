"""The reference-facing classes on the GPU: QKANLayer / QKAN through autograd against golden values."""
import numpy as np
import pytest
import torch

from oracle import oracle
from qkan_b200 import QKAN, QKANLayer, get_solver
from tests.util import GOLDEN, GRAD_NAMES, TOL_BF16, TOL_F32, case_inputs, golden_layer_cases, nerr

pytestmark = pytest.mark.gpu


def _layer_from_case(case, p_dim=4, precise="auto"):
    B, I, O, R = (int(v) for v in case["dims"])
    cfg = case["cfg"]
    layer = QKANLayer(I, O, reps=R, device="cuda", preact_trainable=cfg["preact_trainable"],
                      postact_weight_trainable=True, postact_bias_trainable=cfg["use_postact_bias"],
                      ba_trainable=case["base"], fast_measure=cfg["fast_measure"], p_dim=p_dim,
                      solver_kwargs={"precise": precise})
    with torch.no_grad():
        for name in ("theta", "preacts_weight", "preacts_bias", "postact_weights", "postact_bias",
                     "base_weight", "mask"):
            src = torch.as_tensor(case["in_" + name], dtype=torch.float32, device="cuda")
            getattr(layer, name).copy_(src.reshape(getattr(layer, name).shape))
    layer._mask_is_identity = not case["masked"]
    return layer


@pytest.mark.parametrize("p_dim,precise", [(4, False), (2, "auto")])
@pytest.mark.parametrize("case", golden_layer_cases(), ids=lambda c: c["name"])
def test_layer_autograd_matches_reference(case, p_dim, precise):
    layer = _layer_from_case(case, p_dim, precise).train()
    x = torch.as_tensor(case["in_x"], dtype=torch.float32, device="cuda").requires_grad_(True)
    gy = torch.as_tensor(case["in_gy"], dtype=torch.float32, device="cuda")
    y = layer(x)
    (y * gy).sum().backward()
    assert nerr(y.detach().cpu().numpy(), case["y"]) <= TOL_F32
    assert nerr(x.grad.cpu().numpy(), case["g_x"]) <= TOL_F32
    for name in GRAD_NAMES[1:]:
        p = getattr(layer, name)
        ref = case["g_" + name]
        if p.grad is None:
            assert not p.requires_grad
            continue
        assert nerr(p.grad.reshape(ref.shape).cpu().numpy(), ref) <= TOL_F32, name
    layer.eval()
    with torch.no_grad():
        assert nerr(layer(x).cpu().numpy(), case["y"]) <= TOL_F32
        full = layer.forward_no_sum(x)
    assert nerr(full.sum(dim=2).cpu().numpy(), case["y"]) <= TOL_F32


def test_fit_case_initial_loss_and_gradients_match_reference():
    gold = np.load(f"{GOLDEN}/fit_case.npz")
    xs = torch.as_tensor(gold["train_input"], device="cuda")
    ys = torch.as_tensor(gold["train_label"], device="cuda")
    for tag, ba in (("ba", True), ("noba", False)):
        # seeded initialisation draws from the CPU generator, as in the reference run that made the fixture
        model = QKAN([1, 1], reps=3, seed=0, preact_trainable=True, postact_weight_trainable=True,
                     postact_bias_trainable=True, ba_trainable=ba).to("cuda")
        model.train()
        pred = model(xs)
        loss = torch.nn.functional.mse_loss(pred, ys)
        loss.backward()
        assert nerr(pred.detach().cpu().numpy(), gold[f"{tag}/pred0"]) <= TOL_F32
        assert abs(loss.item() - float(gold[f"{tag}/loss0"])) <= 1e-5 * float(gold[f"{tag}/loss0"])
        for name, p in model.named_parameters():
            key = f"{tag}/grad/{name}"
            if key in gold.files:
                assert nerr(p.grad.cpu().numpy(), gold[key]) <= 2 * TOL_F32, name


def test_fit_case_lbfgs_training_converges_like_the_reference():
    """The 1-D fit of the reference's quick start, 100 LBFGS steps, both base-term settings.

    LBFGS amplifies rounding differences: the reference itself ends at 1.6e-3 or stays on its
    4.5e-3..4.9e-3 plateau depending on the run, so element-wise equality of the trajectory is
    not a meaningful criterion. Checked instead: the first steps follow the reference closely
    and the final losses are within a factor 1.5 of the reference's (its plateau value where
    the reference run that made the fixture left the plateau only late).
    """
    gold = np.load(f"{GOLDEN}/fit_case.npz")
    dataset = {k: torch.as_tensor(gold[k], device="cuda") for k in
               ("train_input", "train_label", "test_input", "test_label")}
    for tag, ba in (("ba", True), ("noba", False)):
        model = QKAN([1, 1], reps=3, seed=0, preact_trainable=True, postact_weight_trainable=True,
                     postact_bias_trainable=True, ba_trainable=ba).to("cuda")
        opt = torch.optim.LBFGS(model.parameters(), lr=5e-2)
        res = model.train_(dataset, optimizer=opt, steps=100, verbose=False)
        assert set(res) == {"train_loss", "test_loss", "reg"} and len(res["train_loss"]) == 100
        ref_train, ref_test = gold[f"{tag}/train_loss"], gold[f"{tag}/test_loss"]
        ours = np.array([float(v) for v in res["train_loss"]])
        assert abs(ours[0] - ref_train[0]) <= 1e-4 * ref_train[0]
        assert abs(ours[1] - ref_train[1]) <= 5e-2 * ref_train[1]
        assert ours[-1] <= 1.5 * max(ref_train[49], ref_train[99]), (tag, ours[-1])
        assert float(res["test_loss"][-1]) <= 1.5 * max(ref_test[49], ref_test[99])
        assert ours[-1] < 0.1 * ours[0]


def test_grouped_theta_and_solver_contract():
    torch.manual_seed(0)
    layer = QKANLayer(6, 4, reps=2, group=3, device="cuda", seed=2, preact_trainable=True,
                      postact_weight_trainable=True, ba_trainable=False)
    x = torch.rand(9, 6, device="cuda") * 2 - 1
    y = layer(x)
    y.square().sum().backward()
    theta, pw, pb = (t.detach().double().cpu().numpy() for t in layer._expanded())
    ones = np.ones((4, 6))
    y_ref = oracle.forward(x.cpu().numpy(), theta, pw, pb, ones, preact_trainable=True)
    assert nerr(y.detach().cpu().numpy(), y_ref) <= TOL_F32
    g = oracle.backward(x.cpu().numpy(), theta, pw, pb, ones, None, None, None, 2 * y_ref, preact_trainable=True)
    g_group = np.stack([g["theta"][:, k::3].sum(axis=(0, 1)) for k in range(3)])
    assert nerr(layer.theta.grad.cpu().numpy(), g_group) <= TOL_F32
    pa = get_solver("b200")(x, layer.theta, layer.preacts_weight, layer.preacts_bias, 2,
                            preacts_trainable=True, fast_measure=True, out_dim=4, group=(3,))
    assert pa.shape == (9, 4, 6)
    assert nerr(pa.sum(dim=2).detach().cpu().numpy(), y_ref) <= TOL_F32


def test_mlp_with_bf16_activations_and_sequence_axis():
    model = QKAN([16, 24, 8], reps=2, seed=4, device="cuda", p_dtype=torch.bfloat16, c_dtype=torch.bfloat16)
    x = (torch.rand(2, 5, 16, device="cuda") * 2 - 1).to(torch.bfloat16)
    y = model(x)
    assert y.shape == (2, 5, 8) and y.dtype == torch.bfloat16
    # float32 twin with the same (bf16-rounded) parameters
    twin = QKAN([16, 24, 8], reps=2, seed=4, device="cuda")
    twin.load_state_dict({k: v.float() for k, v in model.state_dict().items()})
    y32 = twin(x.float())
    assert nerr(y.detach().float().cpu().numpy(), y32.detach().cpu().numpy()) <= 2 * TOL_BF16
    y.float().sum().backward()
    assert all(p.grad is not None and p.grad.dtype == torch.bfloat16
               for p in model.parameters() if p.requires_grad)


def test_host_pipeline_matches_the_direct_call():
    """Chunked, stream-overlapped host-buffer step == one direct call on device-resident tensors."""
    from qkan_b200 import functional as F
    from qkan_b200.host import HostLayerPipeline
    from tests.util import random_problem

    B, I, O, R = 1000, 70, 40, 3
    p = random_problem(11, B, I, O, R, use_pb=True)
    dev = {k: torch.from_numpy(v).cuda() for k, v in p.items() if v is not None}
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    y_ref = F.layer_forward(dev["x"], dev["theta"], dev["pw"], dev["pb"], dev["postw"], dev["postb"], None, None, **cfg)
    g_ref = F.layer_backward(dev["x"], dev["theta"], dev["pw"], dev["pb"], dev["postw"], dev["postb"], None, None,
                             dev["gy"], **cfg)
    pipe = HostLayerPipeline(B, I, O, R, "cuda:0", n_chunks=3)
    hx, hgy = torch.from_numpy(p["x"]).pin_memory(), torch.from_numpy(p["gy"]).pin_memory()
    hy, hgx = torch.empty(B, O).pin_memory(), torch.empty(B, I).pin_memory()
    for _ in range(2):  # the second step reuses the chunk buffers of the first
        bucket = pipe.step(hx, hgy, dev, hy, hgx)
        torch.cuda.synchronize()
        assert nerr(hy.numpy(), y_ref.cpu().numpy()) <= 1e-6
        assert nerr(hgx.numpy(), g_ref["x"].cpu().numpy()) <= 1e-6
        for name in ("theta", "preacts_weight", "preacts_bias", "postact_weights", "postact_bias"):
            assert nerr(bucket[name].cpu().numpy(), g_ref[name].cpu().numpy()) <= 2e-6, name
    # back-to-back steps without a synchronisation in between (copy-out of one step under the next step's
    # kernels), chunk boundaries on multiples of 256 rows, gradients copied to the host as well
    pipe = HostLayerPipeline(B, I, O, R, "cuda:0", n_chunks=4, row_align=256)
    assert [e - b for b, e in pipe.spans] == [256, 256, 256, 232]
    hgrads = torch.empty(pipe.bucket.flat.numel()).pin_memory()
    hy.zero_(), hgx.zero_()
    for _ in range(4):
        bucket = pipe.step(hx, hgy, dev, hy, hgx, hgrads)
    pipe.wait()
    torch.cuda.current_stream().synchronize()
    assert nerr(hy.numpy(), y_ref.cpu().numpy()) <= 1e-6
    assert nerr(hgx.numpy(), g_ref["x"].cpu().numpy()) <= 1e-6
    assert nerr(hgrads.numpy(), bucket.flat.cpu().numpy()) == 0.0


def test_graphed_train_step_and_inference_match_eager():
    """Whole-model CUDA-graph capture (the launch-bound regime): same gradients and outputs as eager."""
    from qkan_b200.graph import make_graphed_inference, make_graphed_train_step

    torch.manual_seed(0)
    model = QKAN([20, 16, 4], reps=2, seed=3, preact_trainable=True, postact_weight_trainable=True).to("cuda")
    x = torch.rand(64, 20, device="cuda") * 2 - 1
    labels = torch.randint(0, 4, (64,), device="cuda")
    loss_fn = torch.nn.functional.cross_entropy
    opt = torch.optim.SGD(model.parameters(), lr=0.0)
    loss_e = loss_fn(model(x), labels)
    loss_e.backward()
    eager = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    step = make_graphed_train_step(model, x, labels, loss_fn, opt)
    for _ in range(2):  # replays are idempotent
        loss_g = step(x, labels)
        torch.cuda.synchronize()
        assert abs(float(loss_g.detach()) - float(loss_e.detach())) <= 1e-6 * abs(float(loss_e.detach()))
        for n, p in model.named_parameters():
            if n in eager:
                assert nerr(p.grad.cpu().numpy(), eager[n].cpu().numpy()) <= 1e-6, n
    # the same step with the gradients gathered into one flat buffer inside the graph (one all-reduce would do)
    flat_step = make_graphed_train_step(model, x, labels, loss_fn, opt, flat_grads=True)
    flat_step(x, labels)
    torch.cuda.synchronize()
    n_trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    assert flat_step.flat.numel() == n_trainable
    for n, p in model.named_parameters():
        if n in eager:
            assert p.grad.data_ptr() >= flat_step.flat.data_ptr()  # a view of the flat buffer
            assert nerr(p.grad.cpu().numpy(), eager[n].cpu().numpy()) <= 1e-6, n
    model.eval()
    with torch.no_grad():
        y_e = model(x)
    infer = make_graphed_inference(model, x)
    x2 = torch.rand_like(x)
    with torch.no_grad():
        y2_e = model(x2)
    assert nerr(infer(x).cpu().numpy(), y_e.cpu().numpy()) <= 1e-6
    assert nerr(infer(x2).cpu().numpy(), y2_e.cpu().numpy()) <= 1e-6


def test_loaded_mask_and_frozen_nonzero_bias_are_honoured():
    """A checkpoint with a pruned mask and a non-zero (frozen) postact_bias must change the output accordingly."""
    torch.manual_seed(1)
    src = QKANLayer(6, 4, reps=2, seed=5, postact_bias_trainable=True, device="cuda")
    with torch.no_grad():
        src.postact_bias.normal_()
        src.mask[1, 2] = 0.0
        src.mask[3, 0] = 0.0
    src._mask_is_identity = False
    dst = QKANLayer(6, 4, reps=2, seed=9, postact_bias_trainable=False, device="cuda")  # bias frozen here
    dst.load_state_dict(src.state_dict())
    assert dst._pb_is_nonzero and not dst._mask_is_identity
    x = torch.rand(10, 6, device="cuda") * 2 - 1
    assert torch.allclose(src(x), dst(x), atol=1e-6)
    ref = oracle.forward(x.cpu().numpy(), *(t.detach().double().cpu().numpy() for t in dst._expanded()),
                         dst.postact_weights.detach().cpu().numpy(), dst.postact_bias.detach().cpu().numpy(),
                         dst.base_weight.detach().cpu().numpy(), dst.mask.detach().cpu().numpy(),
                         preact_trainable=False, use_postact_bias=True)
    assert nerr(dst(x).detach().cpu().numpy(), ref) <= TOL_F32


def test_train_loop_with_adam_pruning_and_grouped_theta():
    """train_ with the default optimiser, theta-magnitude pruning, and grouped theta (pruning must skip it)."""
    torch.manual_seed(0)
    x = torch.rand(256, 3, device="cuda") * 2 - 1
    y = (x[:, :1] * x[:, 1:2] + torch.sin(3 * x[:, 2:3])).contiguous()
    dataset = dict(train_input=x, train_label=y, test_input=x[:128], test_label=y[:128])
    model = QKAN([3, 5, 1], reps=2, seed=1, device="cuda")
    with torch.no_grad():
        model.layers[0].theta[0, 0].zero_()  # one edge below the pruning threshold
    res = model.train_(dataset, steps=6, batch=128, verbose=False, prune_every=2, prune_threshold=1e-6,
                       optimizer=torch.optim.Adam(model.parameters(), lr=1e-2))
    assert len(res["train_loss"]) == 6 and np.isfinite(res["train_loss"]).all()
    assert float(res["train_loss"][-1]) < float(res["train_loss"][0])
    grouped = QKAN([3, 4, 1], reps=2, group=2, seed=1, device="cuda")
    before = [layer.mask.clone() for layer in grouped.layers]
    grouped.train_(dataset, steps=2, verbose=False, prune_every=1, prune_threshold=1e3)
    assert all(torch.equal(a, layer.mask) for a, layer in zip(before, grouped.layers))


@pytest.mark.parametrize("ansatz", ["pz_encoding", "rpz_encoding"])
def test_refine_is_function_preserving(ansatz):
    """Layer extension: the model with more repetitions starts as exactly the same function."""
    torch.manual_seed(0)
    model = QKAN([5, 6, 2], reps=2, seed=4, ansatz=ansatz, preact_trainable=True, ba_trainable=True,
                 postact_bias_trainable=True, device="cuda")
    with torch.no_grad():
        for p in model.parameters():
            if p.requires_grad:
                p.add_(0.1 * torch.randn_like(p))
    x = torch.rand(32, 5, device="cuda") * 2 - 1
    bigger = model.refine(5)
    assert bigger.layers[0].reps == 5 and bigger.layers[0].theta.shape[2] == 6
    assert nerr(bigger(x).detach().cpu().numpy(), model(x).detach().cpu().numpy()) <= 1e-6


@pytest.mark.parametrize("ansatz", ["pz_encoding", "real"])
def test_hybrid_block_bf16_eager_and_graphed(ansatz):
    """Linear -> QKAN -> Linear block in bfloat16: matches a float32 twin, and the captured step matches eager."""
    from qkan_b200 import FusedHQKAN
    from qkan_b200.graph import make_graphed_train_step

    torch.manual_seed(0)
    block = FusedHQKAN(48, 16, reps=2, ansatz=ansatz)
    assert block.qkan.layers[0].solver == "b200" and block.down.weight.dtype == torch.bfloat16
    x = (torch.rand(4, 32, 48, device="cuda") * 2 - 1).to(torch.bfloat16)
    y = block(x.view(-1, 48))
    twin = FusedHQKAN(48, 16, reps=2, ansatz=ansatz, p_dtype=torch.float32, c_dtype=torch.float32)
    twin.load_state_dict({k: v.float() for k, v in block.state_dict().items()})
    y32 = twin(x.view(-1, 48).float())
    assert nerr(y.detach().float().cpu().numpy(), y32.detach().cpu().numpy()) <= 2 * TOL_BF16
    target = torch.randn_like(y)
    loss_fn = lambda out, t: (out.float() - t.float()).square().mean()  # noqa: E731
    loss_e = loss_fn(block(x.view(-1, 48)), target)
    loss_e.backward()
    eager = {n: p.grad.clone() for n, p in block.named_parameters() if p.grad is not None}
    assert "qkan.layers.0.theta" in eager and "down.weight" in eager
    step = make_graphed_train_step(block, x.view(-1, 48), target, loss_fn, torch.optim.SGD(block.parameters(), lr=0.0))
    loss_g = step(x.view(-1, 48), target)
    torch.cuda.synchronize()
    assert abs(float(loss_g.detach()) - float(loss_e.detach())) <= 1e-3 * abs(float(loss_e.detach()))
    for n, p in block.named_parameters():
        if n in eager:
            assert nerr(p.grad.float().cpu().numpy(), eager[n].float().cpu().numpy()) <= 1e-6, n


def test_train_loop_with_a_closure_driven_composite_optimizer():
    """An optimiser that runs Adam first and hands the closure to LBFGS later (the shape of the reference's
    `adam_then_lbfgs`) goes through train_ like LBFGS itself: it gets the built-in closure."""

    class AdamThenLbfgs:
        needs_closure = True

        def __init__(self, params, switch_at):
            self.params, self.switch_at, self.calls = list(params), switch_at, 0
            self.adam = torch.optim.Adam(self.params, lr=1e-2)
            self.lbfgs = None

        def zero_grad(self, set_to_none=True):
            (self.lbfgs or self.adam).zero_grad(set_to_none=set_to_none)

        def step(self, closure):
            self.calls += 1
            if self.calls > self.switch_at and self.lbfgs is None:
                self.lbfgs = torch.optim.LBFGS(self.params, lr=0.5, max_iter=5, line_search_fn="strong_wolfe")
            return (self.lbfgs or self.adam).step(closure)

    torch.manual_seed(0)
    x = torch.rand(300, 2) * 2 - 1
    ds = dict(train_input=x, train_label=(x[:, :1] * x[:, 1:]).sin(), test_input=x, test_label=(x[:, :1] * x[:, 1:]).sin())
    model = QKAN([2, 3, 1], reps=2, seed=0, preact_trainable=True, postact_weight_trainable=True).to("cuda")
    model.device = "cuda"
    opt = AdamThenLbfgs(model.parameters(), switch_at=3)
    res = model.train_(ds, optimizer=opt, steps=6, verbose=False)
    assert len(res["train_loss"]) == 6 and opt.lbfgs is not None
    assert float(res["train_loss"][-1]) < float(res["train_loss"][0])


ACT_SPECS = {
    "mlp_base": dict(width=[5, 4, 3], reps=2, seed=3, ba_trainable=True, save_act=True),
    "mlp_trainable": dict(width=[6, 3, 2], reps=3, seed=5, preact_trainable=True, preact_init=True,
                          postact_weight_trainable=True, postact_bias_trainable=True, save_act=True),
    "born_nobase": dict(width=[4, 5], reps=1, seed=9, fast_measure=False, save_act=True),
}


@pytest.mark.parametrize("name", sorted(ACT_SPECS))
def test_save_act_statistics_and_regulariser_match_reference(name):
    """QKAN.forward(save_act=True): per-layer acts_scale / edge_actscale / subnode_actscale and get_reg against the
    reference's own values (fixture made by tests/golden/make_golden.py), with the per-edge deviations coming from
    the in-kernel statistics instead of a (B, O, I) tensor."""
    gold = np.load(f"{GOLDEN}/act_cases.npz")
    model = QKAN(device="cuda", **ACT_SPECS[name])
    state = {k[len(name) + 7:]: torch.as_tensor(gold[k]) for k in gold.files if k.startswith(name + "/state/")}
    model.load_state_dict(state)
    x = torch.as_tensor(gold[name + "/x"], device="cuda")
    y = model(x)
    assert nerr(y.detach().cpu().numpy(), gold[name + "/y"]) <= TOL_F32
    assert not model.dr_postacts and not model.dr_preacts  # nothing of size (B, O, I) is kept by default
    for l in range(len(model.acts_scale)):
        for key, got in (("acts_scale", model.acts_scale[l]), ("edge_actscale", model.edge_actscale[l]),
                         ("subnode_actscale", model.subnode_actscale[l])):
            want = gold[f"{name}/{key}/{l}"]
            assert nerr(got.detach().cpu().numpy(), want) <= 2e-5, f"{key}[{l}]"
    for metric in ("edge_forward_dr_n", "edge_forward_sum", "edge_forward_dr_u"):
        reg = float(model.get_reg(metric, 1.0, 2.0, 0.1, 0.05))
        want = float(gold[f"{name}/reg/{metric}"])
        assert abs(reg - want) <= 2e-5 * abs(want), metric
    # the opt-in keeps the reference's per-sample edge tensors too
    model.keep_edge_acts = True
    model(x)
    assert model.dr_postacts[0].shape == (x.shape[0], model.width[1], model.width[0])
    assert nerr(torch.std(model.dr_postacts[0], dim=0).cpu().numpy(), gold[f"{name}/edge_actscale/0"]) <= 2e-5


def test_edge_statistics_at_transformer_width_use_no_batch_by_edge_tensor():
    """8192 x 768 -> 768 (the HQKANsformer-shaped layer): the statistics pass peaks at a few hundred MB where
    the (B, O, I) tensor alone would take 19 GB, and agrees with torch.std over forward_no_sum on a slice of outputs."""
    layer = QKANLayer(768, 768, reps=2, device="cuda", ba_trainable=True, seed=1)
    x = torch.randn(8192, 768, device="cuda").clamp_(-3, 3)
    with torch.no_grad():
        layer.postact_weights.mul_(torch.rand_like(layer.postact_weights) + 0.5)
    layer.edge_output_std(x[:64])  # warm the allocator and the kernels
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    got = layer.edge_output_std(x)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - before
    assert peak < 512 * 2**20, f"statistics pass peaked at {peak / 2**20:.0f} MiB"
    outs = [0, 5, 383, 767]
    sub = layer.get_subset(list(range(768)), outs)
    want = torch.std(sub.forward_no_sum(x), dim=0)
    assert nerr(got[outs].cpu().numpy(), want.cpu().numpy()) <= 2e-5
    # ragged batch, bf16 activations
    xb = x[:1000].to(torch.bfloat16)
    gb = layer.edge_output_std(xb)
    wb = torch.std(sub.forward_no_sum(xb.float()), dim=0)
    assert nerr(gb[outs].float().cpu().numpy(), wb.cpu().numpy()) <= 1e-3


@pytest.mark.parametrize("c_dtype", [torch.bfloat16, torch.float8_e4m3fn])
def test_c_dtype_bfloat16_and_float8_run_with_bf16_activations(c_dtype):
    """c_dtype=bfloat16 / float8_e4m3fn: activations cross the kernel boundary as bfloat16, parameters and the result
    keep p_dtype, and values and gradients stay inside the bf16 bound of the float32 layer."""
    kw = dict(reps=3, device="cuda", preact_trainable=True, postact_weight_trainable=True, seed=4)
    ref, low = QKANLayer(24, 16, **kw), QKANLayer(24, 16, c_dtype=c_dtype, **kw)
    x = (torch.rand(200, 24, device="cuda") * 2 - 1)
    xr, xl = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    gy = torch.randn(200, 16, device="cuda")
    yr, yl = ref(xr), low(xl)
    assert yl.dtype == torch.float32
    (yr * gy).sum().backward()
    (yl * gy).sum().backward()
    assert nerr(yl.detach().cpu().numpy(), yr.detach().cpu().numpy()) <= TOL_BF16
    assert nerr(xl.grad.cpu().numpy(), xr.grad.cpu().numpy()) <= TOL_BF16
    for name in ("theta", "preacts_weight", "postact_weights"):
        a, b = getattr(low, name).grad, getattr(ref, name).grad
        assert a.dtype == torch.float32 and nerr(a.cpu().numpy(), b.cpu().numpy()) <= TOL_BF16, name
