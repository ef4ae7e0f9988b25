"""Model definitions used by the benchmarks."""
import torch

from hcomm_b200.models.llama import CONFIGS, Llama


def test_llama_parameter_counts_match_the_published_sizes():
    assert abs(CONFIGS["llama3_8b"].num_params() / 1e9 - 8.03) < 0.01
    assert abs(CONFIGS["llama3_70b"].num_params() / 1e9 - 70.55) < 0.1


def test_tiny_llama_trains_a_step_on_cpu():
    torch.manual_seed(0)
    m = Llama(CONFIGS["tiny"])
    assert sum(p.numel() for p in m.parameters()) == CONFIGS["tiny"].num_params()
    t = torch.randint(0, 512, (2, 17))
    opt = torch.optim.SGD(m.parameters(), lr=0.5)
    first = None
    for _ in range(5):
        opt.zero_grad()
        loss = m(t[:, :-1], t[:, 1:])
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first
