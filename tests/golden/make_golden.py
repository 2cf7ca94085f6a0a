"""Generates tests/golden/layers.npz: seeded inputs and the outputs of independent float64
implementations (PyTorch CPU operators, Hugging Face BertModel) for the layer kinds of the CPU
oracle.  The reference project stores no expected outputs for this path (its DNN tests print ten
values for a human to compare), so these vectors are what the oracle is pinned against when the
libraries that produced them are not installed.

    python tests/golden/make_golden.py        # rewrites tests/golden/layers.npz
"""
import os

import numpy as np
import torch
import torch.nn.functional as F


def main() -> None:
    rng = np.random.default_rng(20240521)
    out = {}

    def t(a):
        return torch.from_numpy(a).double()

    # convolution + bias + residual + ReLU, stride 1 and stride 2
    for tag, (n, cin, h, w, cout, k, stride, pad) in {"conv_s1": (2, 16, 9, 9, 24, 3, 1, 1),
                                                       "conv_s2": (1, 8, 10, 10, 16, 3, 2, 1),
                                                       "conv_1x1": (2, 32, 5, 5, 8, 1, 1, 0)}.items():
        x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
        wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
        b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
        y = F.conv2d(t(x), t(wt), t(b), stride=stride, padding=pad)
        res = rng.standard_normal(tuple(y.shape)).astype(np.float32)
        y = torch.relu(y + t(res)).float().numpy()
        out.update({f"{tag}.x": x, f"{tag}.w": wt, f"{tag}.b": b, f"{tag}.res": res, f"{tag}.y": y,
                    f"{tag}.cfg": np.array([stride, pad], np.int32)})
    # depthwise 3x3 + bias + ReLU6
    x = (rng.standard_normal((2, 16, 7, 7)) * 3).astype(np.float32)
    wt = rng.standard_normal((16, 1, 3, 3)).astype(np.float32)
    b = rng.standard_normal(16).astype(np.float32)
    y = torch.clamp(F.conv2d(t(x), t(wt), t(b), stride=1, padding=1, groups=16), 0.0, 6.0).float().numpy()
    out.update({"dw.x": x, "dw.w": wt, "dw.b": b, "dw.y": y})
    # pooling
    x = rng.standard_normal((2, 8, 13, 11)).astype(np.float32)
    out.update({"pool.x": x, "pool.max3s2p1": F.max_pool2d(t(x), 3, 2, 1).float().numpy(),
                "pool.avg2s2": F.avg_pool2d(t(x[:, :, :12, :10]), 2, 2).float().numpy()})
    x7 = rng.standard_normal((2, 8, 7, 7)).astype(np.float32)
    out.update({"gap.x": x7, "gap.y": F.adaptive_avg_pool2d(t(x7), 1).float().numpy()})
    # one BERT encoder layer (hidden 64, one head, ffn 128) through Hugging Face's BertModel
    from transformers import BertConfig, BertModel

    cfg = BertConfig(vocab_size=50, hidden_size=64, num_hidden_layers=1, num_attention_heads=1,
                     intermediate_size=128, max_position_embeddings=16, hidden_act="gelu",
                     hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(7)
    model = BertModel(cfg, add_pooling_layer=False).double().eval()
    ids = rng.integers(0, 50, (2, 8)).astype(np.int64)
    with torch.no_grad():
        y = model(torch.from_numpy(ids)).last_hidden_state.float().numpy()
    out["bert.ids"] = ids
    out["bert.y"] = y
    for k, v in model.state_dict().items():
        if "position_ids" in k or "token_type_ids" in k:
            continue
        out["bert.param." + k] = v.float().numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "layers.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
