"""The multi-device form of the backend: Backend::create("B200:all") / ("B200:0+1") - the text after ':' is nGraph's backend
option string (src/ngraph/runtime/backend_manager.cpp:83-89,141).  One Backend / Executable / Tensor per logical object;
compile() splits the Function along the batch, every member device runs the same graph on its rows, Tensor::write hands
out rows and Tensor::read collects them.

CPU: the batch split itself (ngraph_b200/backend/batch_split.cpp, no device needed) - the split Function on each slice
gives the rows of the whole Function on the whole batch (INTERPRETER, bit for bit), and graphs that are not independent along
the batch are refused with a reason.  GPU: the same Functions through "B200:0+0" (two members on one device, which a
one-GPU machine can run) and "B200:all" agree with the single-device backend bit for bit, uneven batches included; a
Function that cannot be split runs whole on the first member; tensors move between executables of different kinds."""
import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import interpreter  # noqa: E402

needs_ngraph = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")


def bits(a):
    return a.view(np.uint32) if a.dtype == np.float32 else a


def glue_network(batch):
    """ops the INTERPRETER runs too: a second, batch-free Parameter, a transposing Reshape that keeps the batch in front, a
    flattening Reshape, Dot with constant weights, a broadcast bias row, Softmax over the features"""
    rng = np.random.default_rng(3)
    p = ng.parameter(np.float32, (batch, 16, 6, 6))
    gain = ng.parameter(np.float32, (10,))
    q = ng.quantize(p, np.float32(0.05), np.uint8(128), np.uint8)
    m = ng.max_pool(q, (2, 2), (2, 2))                                  # u8 [B, 16, 3, 3]
    d = ng.dequantize(m, np.float32(0.05), np.uint8(128))
    t = ng.reshape(d, (0, 2, 3, 1), (batch, 3, 3, 16))                  # channels last, batch stays in front
    flat = ng.reshape(t, (0, 1, 2, 3), (batch, 144))
    w = ng.constant(rng.standard_normal((144, 10)).astype(np.float32))
    y = ng.add(ng.dot(flat, w), ng.broadcast(ng.constant(rng.standard_normal(10).astype(np.float32)), (batch, 10), (0,)))
    y = ng.multiply(y, ng.broadcast(gain, (batch, 10), (0,)))
    fn = ng.Function([ng.softmax(y, (1,)), q], [p, gain])
    xs = [rng.standard_normal((batch, 16, 6, 6)).astype(np.float32), rng.uniform(0.5, 1.5, 10).astype(np.float32)]
    return fn, xs


def conv_network(batch, hw=12):
    """the fused quantized ops: conv + bias + relu, MaxPool, conv + bias + residual add, pooling head, QuantizedDot"""
    rng = np.random.default_rng(8)
    shape = (batch, 64, hw, hw)
    w1 = rng.integers(-127, 128, size=(64, 64, 3, 3)).astype(np.int8)
    w2 = rng.integers(-127, 128, size=(64, 64, 1, 1)).astype(np.int8)
    b1 = rng.integers(-500, 500, size=64).astype(np.int32)
    s1 = (np.exp(rng.uniform(-0.5, 0.5, size=64)) * 2e-4).astype(np.float32)
    s2 = (np.exp(rng.uniform(-0.5, 0.5, size=64)) * 6e-4).astype(np.float32)
    wd = rng.integers(-127, 128, size=(64, 10)).astype(np.int8)
    p = ng.parameter(np.float32, shape)
    q = ng.quantize(p, np.float32(0.02), np.uint8(0), np.uint8)
    c1 = ng.quantized_conv_bias(q, w1, b1, s1, True, pad_below=(1, 1))
    mp = ng.max_pool(c1, (3, 3), (2, 2), (1, 1))
    c2 = ng.quantized_conv_bias_add(mp, w2, b1, mp, s2, np.array([0.5], np.float32), True, False)
    pooled = ng.quantize(ng.avg_pool(ng.dequantize(c2, np.float32(0.05), np.uint8(0)), c2.shape[2:]), np.float32(0.04), np.uint8(0), np.uint8)
    flat = ng.reshape(pooled, (0, 1, 2, 3), (batch, 64))
    logits = ng.quantized_dot(flat, ng.constant(wd), 0.04, 0, 0.01, 0, 0.5, 0, np.int8)
    fn = ng.Function([ng.dequantize(logits, np.float32(0.5), np.int8(0)), c2], [p])
    return fn, [rng.standard_normal(shape).astype(np.float32)]


def batch_sum_network(batch):
    """not independent along the batch: a Sum over axis 0"""
    p = ng.parameter(np.float32, (batch, 16))
    fn = ng.Function([ng.reduce_sum(ng.relu(p), (0,))], [p])
    return fn, [np.random.default_rng(5).standard_normal((batch, 16)).astype(np.float32)]


# ---------------------------------------------------------------- CPU: the split
@needs_ngraph
@pytest.mark.parametrize("batch,rows", [(6, 3), (6, 2), (5, 1), (4, 4)])
def test_split_function_reproduces_the_rows_of_the_whole(batch, rows):
    fn, xs = glue_network(batch)
    part, p_split, r_split = ng.split_batch(fn, rows)
    assert p_split == [True, False] and r_split == [True, True]
    assert part.params[0].shape == (rows, 16, 6, 6) and part.params[1].shape == (10,)
    assert part.results[0].shape == (rows, 10) and part.results[1].shape == (rows, 16, 6, 6)
    ref = interpreter.backend()
    whole = ref.compile(fn).run(*xs)
    exe = ref.compile(part)
    for first in range(0, batch - rows + 1, rows):
        got = exe.run(xs[0][first:first + rows], xs[1])
        for g, w in zip(got, whole):
            np.testing.assert_array_equal(bits(g), bits(w[first:first + rows]))


@needs_ngraph
def test_split_keeps_the_fused_quantized_ops():
    fn, _ = conv_network(6)
    part, p_split, r_split = ng.split_batch(fn, 2)
    assert p_split == [True] and r_split == [True, True]
    assert part.params[0].shape == (2, 64, 12, 12) and part.results[0].shape == (2, 10) and part.results[1].shape == (2, 64, 6, 6)
    names = ng.function_op_names(part, lowered=False)
    assert sorted(names) == sorted(ng.function_op_names(ng.after_b200_passes(fn), lowered=False))


@needs_ngraph
def test_graphs_that_mix_samples_are_refused_with_the_reason():
    fn, _ = batch_sum_network(4)
    with pytest.raises(ng.NgraphError, match="reduces over the batch axis"):
        ng.split_batch(fn, 2)
    p = ng.parameter(np.float32, (4, 6))
    with pytest.raises(ng.NgraphError, match="normalises over the batch axis"):
        ng.split_batch(ng.Function([ng.softmax(p, (0,))], [p]), 2)
    with pytest.raises(ng.NgraphError, match="moves the batch axis"):
        ng.split_batch(ng.Function([ng.reshape(p, (1, 0), (6, 4))], [p]), 2)
    with pytest.raises(ng.NgraphError, match="differs between samples"):
        ng.split_batch(ng.Function([ng.add(p, ng.constant(np.arange(24, dtype=np.float32).reshape(4, 6)))], [p]), 2)
    # ... while a constant whose samples are all alike (a folded broadcast) is cut to the rows
    part, _, _ = ng.split_batch(ng.Function([ng.add(p, ng.constant(np.tile(np.arange(6, dtype=np.float32), (4, 1))))], [p]), 2)
    assert part.results[0].shape == (2, 6)
    with pytest.raises(ng.NgraphError, match="does not carry the batch"):
        q = ng.parameter(np.float32, (3,))
        ng.split_batch(ng.Function([ng.relu(p), ng.relu(q)], [p, q]), 2)


@needs_ngraph
def test_dynamic_whole_tensor_scales_keep_the_encoder_on_one_device():
    """the BERT-shaped encoder takes Max(Abs(x)) over all tokens of the batch for its activation scales: a reduction across
    samples, so it is not split"""
    fn = ng.bert_encoder(1, 64, 4, 128, 8, 2, 100)
    with pytest.raises(ng.NgraphError, match="not split"):
        ng.split_batch(fn, 8)


# ---------------------------------------------------------------- GPU
def member_lists():
    import torch
    names = ["B200:0+0", "B200:0+0+0+0+0+0"]  # the second: more members than samples, the last ones stay idle
    if torch.cuda.is_available() and torch.cuda.device_count() >= 2:
        names.append("B200:all")
    return names


@pytest.fixture(scope="module")
def single():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    ng.load_b200()
    return ng.Backend("B200")


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("name", ["B200:0+0", "B200:0+0+0+0+0+0", "B200:all"])
@pytest.mark.parametrize("batch", [4, 5])
def test_split_execution_matches_one_device(single, name, batch):
    from ngraph_b200 import lib
    if name not in member_lists():
        pytest.skip("needs two devices")
    multi = ng.Backend(name)
    for build in (conv_network, glue_network):
        fn, xs = build(batch)
        exp = single.compile(fn).run(*xs)
        exe = multi.compile(fn)
        before = lib.launch_count()
        got = exe.run(*xs)
        launches = lib.launch_count() - before
        for g, e in zip(got, exp):
            np.testing.assert_array_equal(bits(g), bits(e))
        # every member ran the whole step list on its rows
        one = lib.launch_count()
        single.compile(fn).run(*xs)
        one = lib.launch_count() - one
        assert launches >= 2 * one - 2, (launches, one)  # a member with a smaller share may take a different tiling path


@pytest.mark.gpu
@needs_ngraph
def test_executable_made_tensors_are_written_and_read_by_rows(single):
    multi = ng.Backend("B200:0+0")
    fn, xs = conv_network(6)
    exp = single.compile(fn).run(*xs)
    exe = multi.compile(fn)
    t_in = exe.create_input_tensors(0, 2)
    t_out = [exe.create_output_tensors(i, 2) for i in range(2)]
    for k in range(2):  # the pipelined-tensor pattern: two sets in rotation
        t_in[k].write(xs[0])
        exe.call([t_out[0][k], t_out[1][k]], [t_in[k]])
    for k in range(2):
        for i in range(2):
            np.testing.assert_array_equal(bits(t_out[i][k].read()), bits(exp[i]))
    # a tensor from Backend::create_tensor learns its rows at the first call and is refilled by rows afterwards
    t = multi.create_tensor(np.float32, xs[0].shape)
    o = [multi.create_tensor(v.dtype, v.shape) for v in fn.results]
    for _ in range(2):
        t.write(xs[0])
        exe.call(o, [t])
        np.testing.assert_array_equal(bits(o[0].read()), bits(exp[0]))
    # written but never used by a call: read returns what was written
    np.testing.assert_array_equal(t.read(), xs[0])


@pytest.mark.gpu
@needs_ngraph
def test_function_that_cannot_be_split_runs_on_the_first_member(single):
    multi = ng.Backend("B200:0+0")
    fn, xs = batch_sum_network(6)
    exp = single.compile(fn).run(*xs)
    got = multi.compile(fn).run(*xs)
    np.testing.assert_array_equal(bits(got[0]), bits(exp[0]))


@pytest.mark.gpu
@needs_ngraph
def test_tensors_move_between_split_and_whole_executables(single):
    """the rows one executable produced on different members are gathered when the next executable needs the whole tensor"""
    multi = ng.Backend("B200:0+0")
    p = ng.parameter(np.float32, (6, 16))
    first = ng.Function([ng.relu(p)], [p])                       # split: each member holds its rows of the result
    q = ng.parameter(np.float32, (6, 16))
    second = ng.Function([ng.reduce_sum(q, (0,))], [q])          # whole, on the first member
    x = np.random.default_rng(2).standard_normal((6, 16)).astype(np.float32)
    t_x, t_mid, t_out = multi.create_tensor(np.float32, (6, 16)), multi.create_tensor(np.float32, (6, 16)), multi.create_tensor(np.float32, (16,))
    t_x.write(x)
    multi.compile(first).call([t_mid], [t_x])
    multi.compile(second).call([t_out], [t_mid])
    exp = single.compile(second).run(np.maximum(x, 0))[0]
    np.testing.assert_array_equal(bits(t_out.read()), bits(exp))
    # and back: the whole-executable's result (first member only) feeds a split executable
    r = ng.parameter(np.float32, (6, 16))
    third = ng.Function([ng.relu(r)], [r])
    t_whole = multi.create_tensor(np.float32, (6, 16))
    ident = ng.parameter(np.float32, (6, 16))
    whole_fn = ng.Function([ng.add(ident, ng.broadcast(ng.reduce_sum(ident, (0,)), (6, 16), (0,)))], [ident])
    multi.compile(whole_fn).call([t_whole], [t_x])
    t_last = multi.create_tensor(np.float32, (6, 16))
    multi.compile(third).call([t_last], [t_whole])
    exp = single.compile(third).run(single.compile(whole_fn).run(x)[0])[0]
    np.testing.assert_array_equal(bits(t_last.read()), bits(exp))


@pytest.mark.gpu
@needs_ngraph
def test_option_string_errors(single):
    with pytest.raises(ng.NgraphError):
        ng.Backend("B200:0+x")
    with pytest.raises(ng.NgraphError):
        ng.Backend("B200:0+99")
    multi = ng.Backend("B200:0+0")
    with pytest.raises(ng.NgraphError):  # a tensor of the single-device backend is foreign to the multi-device one
        fn, xs = batch_sum_network(4)
        multi.compile(fn).call([single.create_tensor(np.float32, (16,))], [single.create_tensor(np.float32, (4, 16))])


@pytest.mark.gpu
@needs_ngraph
def test_save_and_load_across_the_two_forms(single, tmp_path):
    """a multi-device executable saves the archive of the whole Function; the single-device form loads it as it is, the
    multi-device form rebuilds the Function from it and splits it again"""
    multi = ng.Backend("B200:0+0")
    fn, xs = conv_network(6)
    exp = single.compile(fn).run(*xs)
    path = str(tmp_path / "net.b200")
    multi.compile(fn).save(path)
    for backend in (single, multi):
        got = backend.load(path, fn).run(*xs)
        for g, e in zip(got, exp):
            np.testing.assert_array_equal(bits(g), bits(e))
    # and the other way round: saved by the single-device form, loaded by the multi-device one
    path2 = str(tmp_path / "net_single.b200")
    single.compile(fn).save(path2)
    got = multi.load(path2, fn).run(*xs)
    for g, e in zip(got, exp):
        np.testing.assert_array_equal(bits(g), bits(e))
