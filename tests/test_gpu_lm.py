"""GPU parity of one LSTM language-model training step (config-4 graph at small sizes): the C++
driver over the C ABI against the CPU oracle -- loss, every hidden state, every gradient, and the
parameters after the clipped SGD update."""
import numpy as np
import pytest

from util import assert_close, lm_grad_floors

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("dims,dropout", [
    (dict(V=97, E=32, H=64, L=2, T=4, B=8), 0.2),
    (dict(V=50, E=20, H=12, L=1, T=3, B=5), 0.0),      # odd sizes: every kernel takes its scalar path
    (dict(V=1000, E=128, H=256, L=2, T=6, B=32), 0.2),
])
def test_lm_step_matches_oracle(oracle, dims, dropout, fused):
    from dynet_b200 import lm
    V, E, H, L, T, B = (dims[k] for k in "VEHLTB")
    model = lm.LstmLm(device=0, seed=11, lr=0.1, clip=5.0, dropout=bool(dropout), fused=fused, **dims)
    tokens, masks = lm.synthetic_batch(dims, seed=12, dropout=dropout)
    params = model.params_host()
    loss = model.forward_backward(tokens, masks)
    grads_ref = [np.zeros_like(p) for p in params]
    loss_ref, h_ref = oracle.lstm_lm_fwdbwd((V, E, H, L, T, B), params, grads_ref, tokens,
                                            masks[0] if masks else None, masks[1] if masks else None, want_h=True)
    assert abs(loss - loss_ref) <= 1e-4 * abs(loss_ref)
    assert_close(model.hidden_states_host(), h_ref, 1e-4, floor=0.1, what="hidden states")  # see GEMM_FLOOR in test_gpu_parity.py
    # every embedding row, gate row and vocabulary row is held to its own scale (a wrong rare-word row must fail)
    for k, (got, (want, floor)) in enumerate(zip(model.grads_host(), lm_grad_floors(grads_ref, lm.param_shapes(V, E, H, L)))):
        assert_close(np.asarray(got).reshape(np.shape(want)), want, 1e-4, floor=floor, what="grad of tensor %d (per-row scale)" % k)
    assert model.ctx.device_errors() == 0
    # trainer update (gradient clipping at 5, SimpleSGD lr 0.1) and gradient reset
    p_ref = [p.copy() for p in params]
    oracle.sgd_update(p_ref, grads_ref, 0.1, 5.0)
    model.update()
    for k, (got, want) in enumerate(zip(model.params_host(), p_ref)):
        assert_close(got, want, 1e-5, floor=1e-1, what="param %d after update" % k)
    assert all(float(np.abs(gr).max()) == 0.0 for gr in model.grads_host())
    # second step on the updated parameters, tokens resident on the device this time
    import torch
    tok_dev = torch.from_numpy(tokens.view(np.int32)).cuda()
    md = model.masks_to_device(masks) if masks else None
    model.launch_forward_backward(tok_dev, md)
    loss2 = float(model.loss_dev.item())
    g2 = [np.zeros_like(p) for p in params]
    loss2_ref, _ = oracle.lstm_lm_fwdbwd((V, E, H, L, T, B), p_ref, g2, tokens, masks[0] if masks else None,
                                         masks[1] if masks else None)
    assert abs(loss2 - loss2_ref) <= 1e-4 * abs(loss2_ref)
    model.close()


def test_lm_bad_token_is_reported(oracle):
    from dynet_b200 import capi, lm
    dims = dict(V=20, E=8, H=8, L=1, T=2, B=3)
    model = lm.LstmLm(device=0, seed=1, dropout=False, **dims)
    tokens, _ = lm.synthetic_batch(dims, seed=2, dropout=0.0)
    tokens[1, 1] = 20   # out of range: device-resident ids are clamped and flagged, never dereferenced
    model.forward_backward(tokens, None)
    with pytest.raises(capi.CudaError):
        model.ctx.device_errors()
    model.close()


def test_lm_graph_replay_matches_eager(oracle):
    """The CUDA-graph replay of forward + backward gives bit-identical losses and gradients to issuing the same
    launches one by one (same kernels, same order), on fresh inputs written to the fixed input buffers."""
    import torch
    from dynet_b200 import lm
    dims = dict(V=300, E=64, H=128, L=2, T=5, B=16)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        model = lm.LstmLm(device=0, seed=21, dropout=True, stream=stream.cuda_stream, **dims)
        p0 = model.params_host()
        batches = [lm.synthetic_batch(dims, seed=30 + k, dropout=0.2) for k in range(4)]

        def run(k, update):
            tokens, masks = batches[k]
            loss = model.forward_backward(tokens, masks)
            grads = model.grads_host()
            if update:
                model.update()
            else:
                model.grads.zero_()
            return loss, grads

        eager = [run(k, False) for k in range(4)]          # parameters unchanged: 4 independent problems
        model.set_graph(True)
        replay = [run(k, False) for k in range(4)]         # first call captures, the rest replay
        assert model.graph_launches() > 50
        for (l0, g0), (l1, g1) in zip(eager, replay):
            assert l0 == l1
            for a, b in zip(g0, g1):
                assert np.array_equal(a, b)
        # a replay after a parameter update sees the new weights (the packed copies are refreshed inside the graph)
        run(0, True)
        loss_after, _ = run(1, False)
        p1 = model.params_host()
        g_ref = [np.zeros_like(p) for p in p1]
        tokens, masks = batches[1]
        V, E, H, L, T, B = (dims[k] for k in "VEHLTB")
        loss_ref, _ = oracle.lstm_lm_fwdbwd((V, E, H, L, T, B), p1, g_ref, tokens, masks[0], masks[1])
        assert any(not np.array_equal(a, b) for a, b in zip(p0, p1))
        assert abs(loss_after - loss_ref) <= 1e-4 * abs(loss_ref)
        assert model.ctx.device_errors() == 0
        model.close()


def test_lm_graph_captured_with_a_fresh_parameter_cache_sees_later_updates(oracle):
    """Capture while the cached operand planes of the weights are up to date (eager steps without an update come first),
    then update the parameters and replay: the replay has to split the new weights again.  Sizes at which every product
    runs on the tensor path and reads the cached planes.  The replayed loss and every gradient are compared bit for bit
    with an eager step of a second model that holds the updated parameters, and with the oracle."""
    import torch
    from dynet_b200 import lm
    dims = dict(V=2000, E=256, H=256, L=2, T=4, B=64)
    V, E, H, L, T, B = (dims[k] for k in "VEHLTB")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        model = lm.LstmLm(device=0, seed=23, lr=0.5, clip=50.0, dropout=True, stream=stream.cuda_stream, **dims)
        batches = [lm.synthetic_batch(dims, seed=60 + k, dropout=0.2) for k in range(3)]
        for k in range(2):                       # eager, no update: the parameter cache is filled and stays valid
            model.forward_backward(*batches[k])
            model.grads.zero_()
        model.set_graph(True)
        model.forward_backward(*batches[0])      # captured here, with nothing stale
        model.update()                           # parameters change after the capture
        p1 = model.params_host()
        loss_replay = model.forward_backward(*batches[2])
        g_replay = model.grads_host()
        assert model.graph_launches() > 20
        other = lm.LstmLm(device=0, seed=99, lr=0.5, clip=50.0, dropout=True, stream=stream.cuda_stream, **dims)
        other.set_params_host(p1)
        loss_eager = other.forward_backward(*batches[2])
        g_eager = other.grads_host()
        assert loss_replay == loss_eager
        for k, (a, b) in enumerate(zip(g_replay, g_eager)):
            assert np.array_equal(a, b), "gradient tensor %d: replay differs from an eager step on the updated parameters" % k
        g_ref = [np.zeros_like(p) for p in p1]
        tokens, masks = batches[2]
        loss_ref, _ = oracle.lstm_lm_fwdbwd((V, E, H, L, T, B), p1, g_ref, tokens, masks[0], masks[1])
        assert abs(loss_replay - loss_ref) <= 1e-4 * abs(loss_ref)
        for k, (got, (want, floor)) in enumerate(zip(g_replay, lm_grad_floors(g_ref, lm.param_shapes(V, E, H, L)))):
            assert_close(np.asarray(got).reshape(np.shape(want)), want, 1e-4, floor=floor, what="replayed grad %d (per-row scale)" % k)
        assert model.ctx.device_errors() == 0 and other.ctx.device_errors() == 0
        model.close()
        other.close()


@pytest.mark.parametrize("graph", [False, True])
def test_lm_step_in_phases_equals_the_whole_step(graph):
    """The step split into L + 1 phases (forward + output layer, then one LSTM layer's backward pass each; what a data-parallel
    caller uses to reduce finished gradient buckets early) gives bit for bit the loss and gradients of the one-call step, and
    the gradient ranges the phases report tile the flat buffer."""
    import torch
    from dynet_b200 import lm
    dims = dict(V=2000, E=256, H=256, L=2, T=4, B=64)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        model = lm.LstmLm(device=0, seed=31, dropout=True, stream=stream.cuda_stream, **dims)
        tokens, masks = lm.synthetic_batch(dims, seed=32, dropout=0.2)
        loss_whole = model.forward_backward(tokens, masks)
        g_whole = model.grads_host()
        model.grads.zero_()
        n = model.num_phases()
        assert n == dims["L"] + 1
        ranges = sorted(model.phase_grad_range(p) for p in range(n))
        assert ranges[0][0] == 0 and ranges[-1][0] + ranges[-1][1] == model.n_params
        assert all(a[0] + a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        model.set_graph(graph)
        md = model.masks_to_device(masks)
        for rep in range(2):                       # (graph: captured in the first round, replayed in the second)
            model.grads.zero_()
            final = {}
            for p in range(n):
                model.launch_phase(p, tokens, md)
                off, cnt = model.phase_grad_range(p)
                torch.cuda.synchronize()
                final[p] = model.grads[off:off + cnt].clone()     # must not change in later phases
            loss = float(model.loss_dev.item())
            assert loss == loss_whole
            for a, b in zip(model.grads_host(), g_whole):
                assert np.array_equal(a, b)
            for p in range(n):
                off, cnt = model.phase_grad_range(p)
                assert torch.equal(final[p], model.grads[off:off + cnt])
        assert model.ctx.device_errors() == 0
        model.close()


@pytest.mark.parametrize("rule", ["momentum", "adam"])
def test_lm_training_with_other_trainers(oracle, rule):
    """Three training steps with MomentumSGD / Adam: the gradients come from the LM driver, the clipped update from
    dyb200_squared_norm + dyb200_trainer_update over the flat parameter buffer; the oracle applies the reference's
    update statements tensor by tensor.  Parameters must agree after every step."""
    import torch
    from dynet_b200 import capi, lm
    dims = dict(V=200, E=32, H=64, L=2, T=4, B=16)
    V, E, H, L, T, B = (dims[k] for k in "VEHLTB")
    hp = dict(momentum=dict(lr=0.01, momentum=0.9), adam=dict(lr=0.001, beta_1=0.9, beta_2=0.999, eps=1e-8))[rule]
    nstate = 1 if rule == "momentum" else 2
    model = lm.LstmLm(device=0, seed=5, dropout=False, **dims)
    n = model.params.numel()
    states = [torch.zeros(n, device="cuda") for _ in range(nstate)]
    sumsq = torch.zeros(1, device="cuda")
    p_ref = model.params_host()
    s_ref = [[np.zeros_like(p) for p in p_ref] for _ in range(nstate)]
    for step in range(3):
        tokens, _ = lm.synthetic_batch(dims, seed=40 + step, dropout=0.0)
        model.forward_backward(tokens, None)
        g_ref = [np.zeros_like(p) for p in p_ref]
        oracle.lstm_lm_fwdbwd((V, E, H, L, T, B), p_ref, g_ref, tokens, None, None)
        gscale = oracle.clip_scale(g_ref, 5.0)
        for k in range(len(p_ref)):
            oracle.trainer_update(rule, p_ref[k], g_ref[k], [s[k] for s in s_ref], gscale=gscale, updates=step, **hp)
        hyper = capi.TrainerHyper(hp["lr"], 5.0, 1.0, hp.get("momentum", 0.9), hp.get("eps", 1e-8), 0.95, hp.get("beta_1", 0.9),
                                  hp.get("beta_2", 0.999), step)
        model.ctx.squared_norm(model.grads.data_ptr(), n, sumsq.data_ptr())
        model.ctx.trainer_update(rule, model.params.data_ptr(), model.grads.data_ptr(), [s.data_ptr() for s in states], n, hyper,
                                 sumsq.data_ptr(), zero_grads=True)
        for k, (got, want) in enumerate(zip(model.params_host(), p_ref)):
            assert_close(got, want, 1e-4, floor=1e-1, what="%s: param %d after step %d" % (rule, k, step))
        assert not model.grads_host()[0].any()
    assert model.ctx.device_errors() == 0
    model.close()
