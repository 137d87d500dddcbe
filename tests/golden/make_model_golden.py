#!/usr/bin/env python3
"""Writes tests/golden/model_outputs.npz: outputs of nGraph's INTERPRETER backend (the reference's own kernels, built from
the reference sources by `make -C oracle ref`) on the two whole-model workloads at their own geometry, which take the
INTERPRETER minutes and are therefore computed once here instead of inside every test run:

  resnet50_224_logits  int8 ResNet-50 v1.5 (decomposed graph), ONE 224x224 image: the 1000 f32 logits
  bert768_seq384       one layer of the int8 BERT-base-shaped encoder at full width (hidden 768, 12 heads, FFN 3072) on one
                       sequence of 384 tokens: f32 [384, 768]
  bert768_seq128_b2    the same layer on two sequences of 128 tokens: f32 [256, 768]

The models, seeds and inputs are the ones the tests rebuild (tests/test_resnet50.py, tests/test_bert_encoder.py); the file
also records them.  Usage:  python tests/golden/make_model_golden.py [resnet] [bert]
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
OUT = os.path.join(ROOT, "tests", "golden", "model_outputs.npz")

RESNET = dict(model_seed=0, calibration_batch=2, calibration_size=64, image_seed=11)
BERT = dict(layers=1, hidden=768, heads=12, ffn=3072, vocab=30522)
BERT_CASES = {"bert768_seq384": dict(seq=384, batch=1, input_seed=21, model_seed=5),
              "bert768_seq128_b2": dict(seq=128, batch=2, input_seed=22, model_seed=5)}


def bert_inputs(seq, batch, vocab, seed):
    rng = np.random.default_rng(seed)
    m = batch * seq
    ids = rng.integers(0, vocab, m).astype(np.int32)
    seg = np.zeros((batch, seq), np.int32)
    for b in range(batch):
        seg[b, rng.integers(1, seq):] = 1
    return ids, seg.reshape(m)


def main():
    from ngraph_b200 import ngraph_api as ng
    from oracle import interpreter
    want = set(sys.argv[1:]) or {"resnet", "bert"}
    data = dict(np.load(OUT)) if os.path.exists(OUT) else {}
    ref = interpreter.backend()
    if "resnet" in want:
        from ngraph_b200.harness.resnet50_int8 import QuantizedResNet50, synthetic_images
        model = QuantizedResNet50(seed=RESNET["model_seed"], calibration_batch=RESNET["calibration_batch"],
                                  calibration_size=RESNET["calibration_size"])
        x = synthetic_images(2, RESNET["image_seed"], 224)[:1]
        t = time.time()
        fn, _ = model.build(ng, 1, fused=False, decomposed=interpreter)
        data["resnet50_224_logits"] = ref.compile(fn).run(x)[0]
        print("resnet50 224x224: %.1f s" % (time.time() - t), data["resnet50_224_logits"][0, :4])
    if "bert" in want:
        for name, c in BERT_CASES.items():
            ids, seg = bert_inputs(c["seq"], c["batch"], BERT["vocab"], c["input_seed"])
            t = time.time()
            fn = ng.bert_encoder(seed=c["model_seed"], decomposed=True, seq=c["seq"], batch=c["batch"], **BERT)
            data[name] = ref.compile(fn).run(ids, seg)[0]
            print("%s: %.1f s" % (name, time.time() - t), data[name].shape, float(data[name].std()))
    np.savez_compressed(OUT, **data)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
