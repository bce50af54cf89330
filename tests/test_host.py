"""Host-side mirror of the reference interface: construction, seeded init, state dicts, error behaviour."""
import inspect

import numpy as np
import pytest
import torch

import qkan_b200
from qkan_b200 import QKAN, QKANLayer
from qkan_b200.parallel import GradBucket, layer_grad_shapes, shard_rows
from tests.util import GOLDEN

INIT_SPECS = {
    "fit_1_1": dict(width=[1, 1], reps=3, seed=0),
    "mlp_3_4_2": dict(width=[3, 4, 2], reps=2, seed=7, preact_trainable=True, preact_init=True),
    "pdim2": dict(width=[5, 3], reps=3, seed=3, p_dim=2, ba_trainable=True),
    "map_head": dict(width=[4, 3, 6, 2], reps=1, seed=11, is_map=True, hidden=6),
    "bn_small_gauss": dict(width=[3, 2], reps=2, seed=5, is_batchnorm=True, theta_init="small_gaussian"),
}


@pytest.mark.parametrize("name", sorted(INIT_SPECS))
def test_seeded_init_is_bit_identical_to_the_reference(name):
    gold = np.load(f"{GOLDEN}/init_cases.npz")
    sd = QKAN(**INIT_SPECS[name]).state_dict()
    keys = [k[len(name) + 1:] for k in gold.files if k.startswith(name + "/")]
    assert sorted(keys) == sorted(sd.keys())
    for k in keys:
        assert np.array_equal(sd[k].numpy(), gold[f"{name}/{k}"]), k


def test_constructor_signatures_match_the_reference_defaults():
    layer = inspect.signature(QKANLayer.__init__).parameters
    model = inspect.signature(QKAN.__init__).parameters
    expect_layer = ["in_dim", "out_dim", "reps", "group", "device", "solver", "qml_device", "ansatz",
                    "theta_size", "preact_trainable", "preact_init", "postact_weight_trainable",
                    "postact_bias_trainable", "base_activation", "ba_trainable", "is_batchnorm",
                    "fast_measure", "c_dtype", "p_dtype", "seed", "solver_kwargs", "p_dim",
                    "checkpoint_reps", "theta_init"]
    assert list(layer)[1:] == expect_layer
    assert layer["ba_trainable"].default is True and model["ba_trainable"].default is False
    assert layer["reps"].default == 3 and layer["fast_measure"].default is True
    train = inspect.signature(QKAN.train_).parameters
    assert list(train)[1:8] == ["dataset", "optimizer", "closure", "scheduler", "steps", "log", "loss_fn"]
    assert train["steps"].default == 10 and train["reg_metric"].default == "edge_forward_dr_n"


def test_solver_default_differs_from_the_reference_on_purpose():
    """The reference defaults to solver="exact" (its torch path, src/qkan/qkan.py:106-145); this package has one
    solver and no CPU path, so its default is that solver, and any other name is refused when the layer runs."""
    layer = inspect.signature(QKANLayer.__init__).parameters
    model = inspect.signature(QKAN.__init__).parameters
    assert layer["solver"].default == "b200" and model["solver"].default == "b200"
    l = QKANLayer(3, 2, solver="exact")
    with pytest.raises(NotImplementedError):
        l(torch.zeros(4, 3))


def test_c_dtype_values_the_reference_accepts():
    """complex64/float32: float32 activations; bfloat16 and float8_e4m3fn: bfloat16 activations at the kernel
    boundary (the fp8 value selects state-checkpoint storage in the reference, which this backward does not have);
    anything else is refused instead of being passed through."""
    assert QKANLayer(3, 2).c_dtype == torch.float32 and not QKANLayer(3, 2)._io_bf16
    assert QKANLayer(3, 2, c_dtype=torch.complex128).c_dtype == torch.float64
    assert QKANLayer(3, 2, c_dtype=torch.bfloat16)._io_bf16
    assert QKANLayer(3, 2, c_dtype=torch.float8_e4m3fn)._io_bf16
    assert QKANLayer(3, 2, ansatz="real").c_dtype == torch.bfloat16  # forced by the reference for this ansatz
    with pytest.raises(ValueError):
        QKANLayer(3, 2, c_dtype=torch.int8)


def test_trainable_flags_follow_the_reference():
    l = QKANLayer(3, 2, preact_trainable=False, postact_weight_trainable=True, ba_trainable=False)
    assert not l.preacts_weight.requires_grad and not l.preacts_bias.requires_grad
    assert l.postact_weights.requires_grad and not l.postact_bias.requires_grad
    assert not l.base_weight.requires_grad and float(l.base_weight.abs().sum()) == 0.0
    assert not l.mask.requires_grad


def test_state_dict_round_trip_across_p_dim_and_flag_refresh():
    src = QKANLayer(4, 3, reps=2, seed=1, p_dim=4)
    with torch.no_grad():
        src.mask[0, 1] = 0.0
        src.postact_bias.add_(0.25)
    dst = QKANLayer(4, 3, reps=2, seed=9, p_dim=2)
    dst.load_state_dict(src.state_dict())
    assert dst.theta.shape == (12, 6)
    assert torch.equal(dst._theta_natural(), src.theta)
    assert dst._mask_is_identity is False and dst._pb_is_nonzero is True
    back = QKANLayer(4, 3, reps=2, p_dim=4)
    back.load_state_dict(dst.state_dict())
    assert torch.equal(back.mask, src.mask)


def test_no_cpu_fallback_and_unknown_solver_or_ansatz():
    l = QKANLayer(3, 2, reps=1)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        l(torch.zeros(4, 3))
    with pytest.raises(NotImplementedError):
        QKANLayer(3, 2, solver="exact")(torch.zeros(4, 3))
    with pytest.raises(NotImplementedError):
        QKANLayer(3, 2, ansatz="px_encoding")
    with pytest.raises(ValueError):
        QKANLayer(3, 2, p_dim=3)
    assert "b200" in qkan_b200.get_registry()
    assert qkan_b200.get_solver("b200").name == "b200"


def test_grouped_parameters_are_broadcast_like_the_reference():
    l = QKANLayer(5, 3, reps=2, group=2, seed=0, preact_trainable=True)
    assert l.theta.shape == (2, 3, 2)
    theta, pw, pb = l._expanded()
    assert theta.shape == (3, 5, 3, 2) and pw.shape == (3, 5, 2)
    for i in range(5):
        assert torch.equal(theta[1, i], l.theta[i % 2])


def test_shard_rows_covers_every_row_once():
    for n, w in ((65536, 8), (10, 3), (2, 4), (0, 2)):
        spans = [shard_rows(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1


def test_grad_bucket_views_alias_one_flat_buffer():
    shapes = layer_grad_shapes(5, 3, 2)
    bucket = GradBucket(shapes, "cpu")
    assert list(shapes) == ["theta", "preacts_weight", "preacts_bias", "postact_weights", "postact_bias"]
    bucket["theta"].fill_(2.0)
    bucket["postact_bias"].fill_(3.0)
    assert float(bucket.flat.sum()) == 2.0 * 3 * 5 * 3 * 2 + 3.0 * 15
    assert all(bucket.offsets[k] % 64 == 0 for k in shapes)
    bucket.all_reduce()  # no process group: a no-op


def test_parameter_shapes_of_the_other_ansaetze_follow_the_reference():
    rpz = QKANLayer(4, 3, reps=2, ansatz="rpz_encoding")
    assert rpz.theta.shape == (3, 4, 3, 1)
    assert rpz.preacts_bias.requires_grad and not rpz.preacts_weight.requires_grad
    real = QKANLayer(4, 3, reps=2, ansatz="real", p_dim=2)
    assert real.theta.shape == (12, 2) and real._theta_natural().shape == (3, 4, 2, 1)
    assert real.c_dtype == torch.bfloat16


def test_refine_copies_the_leading_circuit_layers_and_zeroes_the_rest():
    """Layer extension (reference: src/qkan/qkan.py:1315-1445): old layers first, added layers at zero angles."""
    small = QKAN([3, 4, 2], reps=2, seed=1, preact_trainable=True, is_map=True, hidden=3)
    with torch.no_grad():
        for p in small.parameters():
            p.add_(0.25)
    big = small.layer_extension(4)
    assert big.reps == 4 and list(big.width) == list(small.width)
    for dst, src in zip(big.layers, small.layers):
        if isinstance(dst, QKANLayer):
            assert dst.reps == 4 and tuple(dst.theta.shape) == (dst.out_dim, dst.in_dim, 5, 2)
            assert torch.equal(dst.theta[:, :, :3], src.theta)
            assert not dst.theta[:, :, 3:].any()
            assert torch.equal(dst.preacts_weight[..., :2], src.preacts_weight)
            assert torch.equal(dst.preacts_bias[..., :2], src.preacts_bias)
            for name in ("postact_weights", "postact_bias", "base_weight"):
                assert torch.equal(getattr(dst, name), getattr(src, name))
        elif isinstance(dst, torch.nn.Linear):
            assert torch.equal(dst.weight, src.weight) and torch.equal(dst.bias, src.bias)
    with pytest.raises(AssertionError):
        small.refine(2)
    with pytest.raises(AssertionError):
        QKAN([3, 5, 2], reps=4).initialize_from_another_model(small)
    assert not big.initialize_parameters().layers[0].theta.any()


def test_host_pipeline_chunks_cover_the_batch_in_whole_waves():
    from qkan_b200.host import chunk_spans

    wave = 148 * 64
    spans = chunk_spans(65536, 3)
    assert spans == [(0, 3 * wave), (3 * wave, 6 * wave), (6 * wave, 65536)]
    assert chunk_spans(65536, 4) == [(0, 2 * wave), (2 * wave, 4 * wave), (4 * wave, 6 * wave), (6 * wave, 65536)]
    assert chunk_spans(1000, 4, row_align=256) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert chunk_spans(1000, 3) == [(0, 334), (334, 668), (668, 1000)]  # too small to align: equal chunks
    assert chunk_spans(5, 8) == [(i, i + 1) for i in range(5)] and chunk_spans(0, 4) == []
    for batch, n in ((1, 1), (9472, 2), (100000, 5), (65537, 3)):
        s = chunk_spans(batch, n)
        assert s[0][0] == 0 and s[-1][1] == batch and len(s) <= n
        assert all(a[1] == b[0] for a, b in zip(s, s[1:]))


def test_host_thread_binding_is_a_no_op_without_a_gpu():
    import os

    from qkan_b200 import bind_host_thread_near_gpu

    before = os.sched_getaffinity(0)
    assert bind_host_thread_near_gpu(0) is None or isinstance(bind_host_thread_near_gpu(0), int)
    assert os.sched_getaffinity(0) <= before  # never widens the mask; unchanged when NVML has no device
