"""The forecast of the memory a model takes (weights, cache, scratch) and the refusal before anything is
allocated."""
import pytest
import torch

from helpers import TINY, cpu_model, model_folder


def test_forecast_counts_what_is_allocated():
    m = cpu_model("B", "float32", max_tokens=640)
    fc = m.forecast(640)
    cfg = TINY["B"]
    # weights: every tensor of the plan; float32 path keeps 4 bytes per element
    plan_bytes = 0
    for spec in m.plan().values():
        n = 1
        for d in spec.shape:
            n *= d
        plan_bytes += n * 4
    assert fc.weights == plan_bytes
    # cache: layers x pages x (k, v) x kv heads x 64 x head_dim x 4 bytes; the model's cache holds exactly that
    pages = 640 // 64
    assert fc.cache == cfg["num_hidden_layers"] * pages * 2 * cfg["num_key_value_heads"] * 64 * cfg["head_dim"] * 4
    from cima_b200.sampling import sampler_state
    with_state = m.forecast(640, extra_state=sampler_state())      # as load_model asks: the sampler's state per slot
    assert with_state.cache == (sum(g.nbytes() for g in m.cache.groups)
                                + sum(t.numel() * t.element_size() for t in m.cache.state.values()))
    assert fc.scratch > 0 and fc.total == fc.weights + fc.cache + fc.scratch
    assert "GiB" in fc.describe()
    half = cpu_model("B", "bfloat16", max_tokens=640).forecast(640)
    assert half.cache * 2 == fc.cache          # bfloat16 keys and values


@pytest.mark.gpu
def test_a_cache_that_cannot_fit_is_refused_before_allocating():
    from cima_b200.engine import load_model
    from cima_b200.engine.fit import DoesNotFit
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    with pytest.raises(DoesNotFit, match="does not fit"):
        load_model(model_folder("B"), dtype="bfloat16", max_tokens=10 ** 10, device="cuda:0", verbose=False)
    assert torch.cuda.memory_allocated() == before


def test_how_far_prompt_steps_are_recorded_follows_the_model_size():
    """A recorded prompt step pays while the device finishes its padded rows before the host could have issued the
    launches: the known shapes land where they were measured to (0.5B wins up to 2,048 rows, 1.5B up to 768, 3B up to
    512 or 768, 7B and larger only within the 256 rows that every model gets)."""
    from cima_b200.config.shapes import SHAPES
    from cima_b200.engine.graph import PROMPT_ROWS, recorded_prompt_rows

    def step_bytes(c):
        H, I, L = c["hidden_size"], c["intermediate_size"], c["num_hidden_layers"]
        qkv = (c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"]
        return 2 * (L * (H * qkv + c["num_attention_heads"] * c["head_dim"] * H + 3 * H * I) + c["vocab_size"] * H)

    got = {name: recorded_prompt_rows(step_bytes(SHAPES[name]), SHAPES[name]["num_hidden_layers"], 2)
           for name in ("qwen2.5-0.5b", "qwen2.5-1.5b", "qwen2.5-3b", "qwen2.5-7b", "qwen2.5-32b")}
    assert got == {"qwen2.5-0.5b": 2048, "qwen2.5-1.5b": 768, "qwen2.5-3b": 512, "qwen2.5-7b": PROMPT_ROWS,
                   "qwen2.5-32b": PROMPT_ROWS}
    assert recorded_prompt_rows(1e6, 2, 4) == 2048 and recorded_prompt_rows(1e12, 2, 2) == PROMPT_ROWS
