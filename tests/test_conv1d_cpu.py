"""The PyTorch statement of the causal convolution op (the oracle of the CUDA kernels): plain rows, packed documents, activation."""
import torch

from surogate_b200.ops.conv1d import causal_conv1d, causal_conv1d_reference


def test_reference_forms_agree_and_respect_document_boundaries():
    torch.manual_seed(0)
    B, T, C, K = 2, 20, 16, 4
    x, w, b = torch.randn(B, T, C), torch.randn(C, K), torch.randn(C)
    plain = causal_conv1d_reference(x, w, b)
    one_doc = causal_conv1d_reference(x, w, b, seq_id=torch.zeros(B, T, dtype=torch.int32))
    assert torch.allclose(plain, one_doc, atol=1e-6)
    want = torch.zeros(B, T, C)
    for t in range(T):
        for k in range(K):
            s = t - (K - 1) + k
            if s >= 0:
                want[:, t] += x[:, s] * w[:, k]
    assert torch.allclose(plain, want + b, atol=1e-5)
    ids = torch.zeros(B, T, dtype=torch.int32)
    ids[:, 7:] = 1
    ids[:, 15:] = 2
    packed = causal_conv1d_reference(x, w, b, "silu", ids)
    for lo, hi in ((0, 7), (7, 15), (15, 20)):           # every document equals the convolution of that document alone
        alone = causal_conv1d_reference(x[:, lo:hi], w, b, "silu")
        assert torch.allclose(packed[:, lo:hi], alone, atol=1e-5)
    assert torch.equal(causal_conv1d(x, w, b), plain)    # on the CPU the public entry is the reference
