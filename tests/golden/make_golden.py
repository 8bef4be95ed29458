"""Extracts the known-answer vectors that SharpNet's own tests hold for the Dot / Dense path and
writes them to ``reference_vectors.json`` next to this script.

Run it where a checkout of the reference is available:
    python tests/golden/make_golden.py /path/to/SharpNet
Nothing at test or run time reads the reference: the JSON file is committed.

Sources (paths inside the reference):
  Tests/GPU/TestGpuTensor.cs:50-120              exact Dot cases (tolerance 1e-9)
  Tests/NonReg/TestNetworkPropagation.cs:24-34   inputs X_1_1_4_4, X_2_1_4_4 and weights W_N_1_4_4
  Tests/NonReg/TestNetworkPropagation.cs:80-132  Linear + Sigmoid predictions before training and after 10 epochs of
                                                 VanillaSGD ([in,out] weights)
  Tests/NonReg/TestNetworkPropagation.cs:135-160,216-244,330-358,725-770,1161-1192
                                                 Linear networks with Softmax, ReLU, LeakyRelu, weight decay and Mse loss:
                                                 predictions before training and after 10 epochs
  Tests/NonReg/TestNetworkPropagation.cs:500-575 attention block: predictions before training, plain and causal
  Tests/NonReg/TestNetworkPropagation.cs:580-623 MultiHeadAttention (3 heads x 5, [in,out] weights): predictions before
                                                 training and after 10 epochs of SGD with momentum, plain and causal
  Tests/NonReg/ParallelRunWithPyTorch.cs:963-1010 ScaledDotProductAttention without scaling ([out,in] weights), plain and
                                                 causal: CategoricalCrossentropy loss before training and after 10 epochs
                                                 of SGD with momentum and weight decay in batches of 2
  Tests/NonReg/ParallelRunWithPyTorch.cs:1013-1129 MultiHeadAttention (3 heads x 2, [out,in] weights), with and without
                                                 bias, plain and causal: CategoricalCrossentropy loss before training
                                                 and after 10 epochs of SGD with momentum in batches of 2
  Tests/NonReg/ParallelRunWithPyTorch.cs:102-138 Linear(5->3, last-dim flatten)+ReLU+Flatten+Linear(36->3), Mse
  Tests/NonReg/ParallelRunWithPyTorch.cs:179-214 Linear(16->3)+ReLU+Linear(3->3)+Sigmoid, BCE ([out,in] weights)
  Tests/NonReg/ParallelRunWithPyTorch.cs:813-850 Linear(16->3)+LeakyRelu(0.1)+Linear(3->3)+Softmax, 10 rows in batches of 2
  (for the three PyTorch-layout networks also the loss after 10 epochs of SGD with momentum / weight decay / Nesterov)
"""
import json
import os
import re
import sys


def _between(text, start_marker, end_marker):
    i = text.index(start_marker)
    j = text.index(end_marker, i)
    return text[i:j]


def _numbers(s):
    return [float(v) for v in re.findall(r"-?\d+\.?\d*(?:[eE]-?\d+)?", s)]


def _const(text, name):
    m = re.search(name + r'\s*=\s*@?"(.*?)";', text)
    body = m.group(1)
    body = body.replace("numpy.array(", "").replace(", numpy.float)", "")
    return _numbers(body)


def _nth_numpy_literal(block, n):
    lits = re.findall(r'FromNumpyArray\("(\[\[.*?\]\])"\)', block)
    return _numbers(lits[n])


def main(ref):
    out = {}
    # ---- exact Dot cases: (aShape, a, bShape, b, expectedShape, expected) -------------------
    gpu = open(os.path.join(ref, "Tests/GPU/TestGpuTensor.cs"), encoding="utf-8-sig").read()
    block = _between(gpu, "public void TestDot()", "// [10x1x28x28]")
    cases = []
    # Walk the block statement by statement instead of trusting regex order.
    stmts = [s.strip() for s in block.split(";")]
    cur = {}
    last_data = None
    for s in stmts:
        m = re.search(r"float\[\]\s+(\w+)\s*=\s*new\s*\[\]\s*\{(.*?)\}", s, re.S)
        if m:
            last_data = [float(v.strip().rstrip("f")) for v in m.group(2).split(",") if v.strip()]
            cur[m.group(1)] = last_data
            continue
        m = re.search(r"(\w+)\s*=\s*new GPUTensor<float>\(new\s*\[\]\s*\{(.*?)\},\s*(\w+),", s, re.S)
        if m:
            name, shape, data = m.group(1), [int(v) for v in m.group(2).split(",")], m.group(3)
            cur[("t", name.split()[-1])] = (shape, cur.get(data))
            continue
        m = re.search(r"expected\s*=\s*new CpuTensor<float>\(new\s*\[\]\s*\{(.*?)\},\s*new\s*\[\]\s*\{(.*?)\}\)", s, re.S)
        if m:
            eshape = [int(v) for v in m.group(1).split(",")]
            edata = [float(v.strip().rstrip("f")) for v in m.group(2).split(",") if v.strip()]
            a_shape, a = cur[("t", "a")]
            b_shape, b = cur[("t", "b")]
            cases.append({"a_shape": a_shape, "a": a, "b_shape": b_shape, "b": b, "expected_shape": eshape,
                          "expected": edata})
    out["dot_exact"] = cases
    out["dot_exact_zero_cases"] = [
        {"a_shape": [10, 1, 28, 28], "b_shape": [784, 100], "expected_shape": [10, 1, 1, 100]},
        {"a_shape": [35, 124], "b_shape": [124, 21], "expected_shape": [35, 21]},
    ]

    # ---- Keras-layout network goldens --------------------------------------------------------
    tnp = open(os.path.join(ref, "Tests/NonReg/TestNetworkPropagation.cs"), encoding="utf-8-sig").read()
    out["X_1_1_4_4"] = _const(tnp, "X_1_1_4_4")
    out["X_2_1_4_4"] = _const(tnp, "X_2_1_4_4")
    out["W_N_1_4_4"] = _const(tnp, "W_N_1_4_4")          # [16, 3]  = [in, out]
    blk = _between(tnp, "public void TestSigmoidActivation_NCHW_1_1_4_4", "const int num_epochs")
    out["sigmoid_1_1_4_4_pred"] = _numbers(re.search(r'TestPredict\(network, X, "(.*?)"\)', blk).group(1))
    out["sigmoid_1_1_4_4_loss"] = _numbers(re.search(r"TestLossAccuracy\(network, X, Y, ([0-9.]+)", blk).group(1))[0]
    blk = _between(tnp, "public void TestSigmoidActivation_NCHW_2_1_4_4", "const int num_epochs")
    out["sigmoid_2_1_4_4_pred"] = _numbers(re.search(r'TestPredict\(network, X, "(.*?)"\)', blk).group(1))
    out["sigmoid_2_1_4_4_loss"] = _numbers(re.search(r"TestLossAccuracy\(network, X, Y, ([0-9.]+)", blk).group(1))[0]
    # predictions and loss after 10 epochs of VanillaSGD (lr 0.1, TensorFlow compatibility mode): pins dW, db, update
    for key in ("1_1_4_4", "2_1_4_4"):
        blk = _between(tnp, "public void TestSigmoidActivation_NCHW_" + key, "public void Test" + ("SigmoidActivation_NCHW_2_1_4_4" if key == "1_1_4_4" else "SoftmaxActivation_NCHW_2_1_4_4"))
        after = blk[blk.index("//predictions after training"):]
        out[f"sigmoid_{key}_pred_after"] = _numbers(re.search(r'TestPredict\(network, X, "(.*?)"\)', after).group(1))
        out[f"sigmoid_{key}_loss_after"] = _numbers(re.search(r"TestLossAccuracy\(network, X, Y, ([0-9.]+)", after).group(1))[0]
    blk = _between(tnp, "public void TestSigmoidActivation_NCHW_1_1_1_1", "const int num_epochs")
    out["sigmoid_1_1_1_1_w"] = _nth_numpy_literal(blk, 0)
    out["sigmoid_1_1_1_1_pred"] = _numbers(re.search(r'TestPredict\(network, X, "(.*?)"\)', blk).group(1))

    # ---- more Dense networks of the same file, each with predictions (and losses where the test states them)
    #      before training and after 10 epochs on the one batch of 2 rows -----------------------------------------
    out["Y_2_3"] = _const(tnp, "Y_2_3")
    out["X_2_3_4_5"] = _const(tnp, "X_2_3_4_5")

    def network_case(name, end):
        blk = _between(tnp, "public void " + name, end)
        weights = [_numbers(c) for c in re.findall(r'FromNumpyArray\("(\[\[.*?\]\])"\)', blk)
                   if len(_numbers(c)) > 6]                      # weight literals (predictions have 6 numbers)
        preds = [_numbers(c) for c in re.findall(r'TestPredict\(network, X,\s*"(.*?)"', blk)]
        losses = [float(v) for v in re.findall(r"TestLossAccuracy\(network, X, Y, ([0-9.]+),", blk)]
        hidden = [float(v) for v in re.findall(r"TestLossAccuracy\(network, X, Y, null\s*/\*\s*([0-9.]+)\s*\*/", blk)]
        return {"weights": weights, "pred_before": preds[0], "pred_after": preds[1],
                "loss_before": (losses or hidden or [None])[0], "loss_after": (losses or hidden or [None, None])[1]}
    # :135-160 Linear(3) + Softmax, CategoricalCrossentropy, VanillaSGD lr 0.1
    out["softmax_2_1_4_4"] = network_case("TestSoftmaxActivation_NCHW_2_1_4_4", "public static CpuTensor<float> FromNumpyArray")
    # :216-244 Linear(3) + ReLU + Linear(3) + Sigmoid, BinaryCrossentropy, VanillaSGD lr 0.1
    out["relu_2_1_4_4"] = network_case("TestReluActivation_NCHW_2_1_4_4", "public void TestEmbedding(")
    # :330-358 Linear(3) + LeakyRelu(0.1) + Linear(3) + Sigmoid, BinaryCrossentropy, SGD lr 0.1 momentum 0.9
    out["leaky_relu_2_1_4_4"] = network_case("TestLeakyReluActivation_NCHW_2_1_4_4", "public void TestConvolutionWithReluActivation")
    # :725-770 Linear(3) + Softmax with weight decay: VanillaSGD lr 0.12, weight_decay 0.05; SGD lr 0.12 momentum 0.9,
    # weight_decay 0.5 (the losses there are commented out in the reference: they include the regularisation term)
    out["weight_decay_vanilla_2_1_4_4"] = network_case("Test_weight_decay_LinearLayer_SGDVanilla_NCHW_2_1_4_4",
                                                       "public void Test_weight_decay_LinearLayer_SGDMomentum")
    out["weight_decay_momentum_2_1_4_4"] = network_case("Test_weight_decay_LinearLayer_SGDMomentum_NCHW_2_1_4_4",
                                                        "public void TestConcatenate_NCHW_1_1_1_1")
    # :1161-1192 Linear(3, on the last dimension) + ReLU + Linear(3), Mse, SGD lr 0.1 momentum 0.9; tolerance 1e-3
    out["mse_2_3_4_5"] = network_case("Test_MseLoss", "private const string X_RNN_4_2_1")

    # ---- attention goldens: Conv1D(k=1) Q/K/V projections -> ScaledDotProductAttention -> Flatten -> Linear -> Softmax
    out["X_3_4_5"] = _const(tnp, "X_3_4_5")
    for name, key in (("Test_ScaledDotProductAttention(", "sdpa"), ("Test_ScaledDotProductAttention_with_Causal_Mask(", "sdpa_causal")):
        blk = _between(tnp, "public void " + name, "TestNetwork.Fit")
        convs = re.findall(r'FromTensorFlowConvNumpyArray\("(.*?)"\)', blk)
        out[key + "_wq"], out[key + "_wk"], out[key + "_wv"] = (_numbers(c) for c in convs)      # each [4 in, 2 out]
        out[key + "_wlinear"] = _numbers(re.findall(r'FromNumpyArray\("(\[\[.*?\]\])"\)\.CopyTo', blk)[0])   # [10, 3]
        out[key + "_pred"] = _numbers(re.search(r'TestPredict\(network, X, "(.*?)"\)', blk).group(1))

    # ---- multi-head attention, Keras layout: Conv1D(k=1) Q/K/V -> MultiHeadAttention(3 heads, key_dim 5) -> Flatten
    #      -> Linear(30 -> 3, [in, out]) -> Softmax on X = numpy_array_for_tests(3, 7, 15)
    i = tnp.index("public void Test_MultiHeadAttention_GPU")
    blk = tnp[i:tnp.index("//predictions before training", i)]
    head = tnp[tnp.rindex("[TestCase(false, false, false", 0, i):i]
    convs = re.findall(r'FromTensorFlowConvNumpyArray\("(.*?)"\)', blk)
    lits = re.findall(r'FromNumpyArray\("(\[\[.*?\]\])"\)\.CopyTo', blk)
    out["mha_tf"] = {
        "conv_q": _numbers(convs[0]), "conv_k": _numbers(convs[1]), "conv_v": _numbers(convs[2]),     # [7 in, 2 out]
        "w_q": _numbers(lits[0]), "w_k": _numbers(lits[1]), "w_v": _numbers(lits[2]),                 # [15 in, 3 x 5 out]
        "w_o": _numbers(lits[3]), "w_linear": _numbers(lits[4]),                                      # [15, 15], [30, 3]
        "cases": [{"use_bias": c[0] == "true", "causal": c[2] == "true", "pred_before": _numbers(c[3]),
                   "pred_after": _numbers(c[4])}     # after 10 epochs of SGD (lr 0.01, momentum 0.9), one batch of 3
                  for c in re.findall(r'\[TestCase\((\w+), (\w+), (\w+), "(.*?)", "(.*?)"\)', head)],
    }

    # ---- PyTorch-layout network goldens ------------------------------------------------------
    pt = open(os.path.join(ref, "Tests/NonReg/ParallelRunWithPyTorch.cs"), encoding="utf-8-sig").read()
    # multi-head attention, PyTorch layout: Conv1D(k=1) Q/K/V ([out, in, 1]) -> MultiHeadAttention(3 heads, key_dim 2,
    # in_proj_weight [18, 6] = w_Q | w_K | w_V, out_proj_weight [6, 6]) -> Flatten -> Linear(12 -> 3, [out, in]) -> Softmax
    # on X = numpy_array_for_tests(10, 2, 6), Y = y_numpy_array_for_tests(10, 3)
    for name in ("no_bias", "with_bias"):
        i = pt.index("public void Test_MultiHeadAttention_" + name)
        blk = pt[i:pt.index("Train(model, X, Y)", i)]
        head = pt[pt.rindex("[TestCase(false", 0, i):i]
        lits = [_numbers(c) for c in re.findall(r'FromNumpyArray\("(\[\[.*?\]\])"\)\.CopyTo', blk)]
        out["mha_pt_" + name] = {
            "conv_q": lits[0], "conv_k": lits[1], "conv_v": lits[2], "in_proj_weight": lits[3], "out_proj_weight": lits[4],
            "w_linear": lits[5],
            "cases": [{"causal": c[0] == "true", "loss_before": float(c[1]), "loss_after": float(c[2])}
                      for c in re.findall(r"\[TestCase\((\w+), ([0-9.]+), ([0-9.]+)\)", head)],
        }
    # :963-1010 Conv1D(k=1) Q/K/V ([2 out, 4 in, 1]) -> ScaledDotProductAttention(no scaling, plain / causal) -> Flatten ->
    # Linear(10 -> 3, [out, in]) -> Softmax on X = numpy_array_for_tests(6, 4, 5): CategoricalCrossentropy before training
    # and after 10 epochs of SGD (lr 0.1, momentum 0.9, weight decay 0.07) in batches of 2
    i = pt.index("public void Test_DotProductAttention(")
    blk = pt[i:pt.index("Train(model, X, Y)", i)]
    head = pt[pt.rindex("[TestCase(false", 0, i):i]
    lits = [_numbers(c) for c in re.findall(r'FromNumpyArray\("(\[\[.*?\]\])"\)\.CopyTo', blk)]
    out["sdpa_pt"] = {"conv_q": lits[0], "conv_k": lits[1], "conv_v": lits[2], "w_linear": lits[3],
                      "cases": [{"causal": c[0] == "true", "loss_before": float(c[1]), "loss_after": float(c[2])}
                                for c in re.findall(r"\[TestCase\((\w+), ([0-9.]+), ([0-9.]+)\)", head)]}
    blk = _between(pt, "public void TestParallelRunWithPyTorch_Mse()", "public void TestParallelRunWithPyTorch_Mse_AdamW")
    out["pt_mse_w1"] = _nth_numpy_literal(blk, 0)         # [3, 5]  = [out, in]
    out["pt_mse_w2"] = _nth_numpy_literal(blk, 1)         # [3, 36]
    out["pt_mse_loss_before"] = _numbers(re.search(r"Assert.AreEqual\(([0-9.]+), loss_before", blk).group(1))[0]
    blk = _between(pt, "public void TestReluActivation_NCHW_2_1_4_4()", "//test_save_sharpnet")
    out["pt_relu_w1"] = _nth_numpy_literal(blk, 0)        # [3, 16]
    out["pt_relu_w2"] = _nth_numpy_literal(blk, 1)        # [3, 3]
    out["pt_relu_loss_before"] = _numbers(re.search(r"Assert.AreEqual\(([0-9.]+), loss_before", blk).group(1))[0]
    out["pt_relu_loss_after"] = _numbers(re.search(r"Assert.AreEqual\(([0-9.]+), loss_after", blk).group(1))[0]
    blk = _between(pt, "public void TestParallelRunWithPyTorch_Mse()", "public void TestParallelRunWithPyTorch_Mse_AdamW")
    out["pt_mse_loss_after"] = _numbers(re.search(r"Assert.AreEqual\(([0-9.]+), loss_after", blk).group(1))[0]
    # :813-850 Flatten + Linear(16->3) + LeakyRelu(0.1) + Linear(3->3) + Softmax on 10 rows in batches of 2,
    # CategoricalCrossentropy, SGD lr 0.1 momentum 0.66 weight_decay 0.17 Nesterov, PyTorch compatibility mode
    blk = _between(pt, "public void TestLeakyReluActivation_NCHW_10_1_4_4()", "public void TestMultiply_NCHW_2_3_4_5_different_dimension")
    out["pt_leaky_w1"] = _nth_numpy_literal(blk, 0)       # [3, 16]
    out["pt_leaky_w2"] = _nth_numpy_literal(blk, 1)       # [3, 3]
    out["pt_leaky_loss_before"] = _numbers(re.search(r"Assert.AreEqual\(([0-9.]+), loss_before", blk).group(1))[0]
    out["pt_leaky_loss_after"] = _numbers(re.search(r"Assert.AreEqual\(([0-9.]+), loss_after", blk).group(1))[0]

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", dst, {k: (len(v) if isinstance(v, list) else v) for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/SharpNet")
    main(sys.argv[1])
