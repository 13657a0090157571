"""The memory plan's arithmetic against sizes worked out by hand for configuration B."""
import pytest
import torch

from helpers import TINY_B
from vllm_cpp_b200 import EngineConfig
from vllm_cpp_b200.config.engine_config import ConfigError
from vllm_cpp_b200.config.registry import resolve_architecture
from vllm_cpp_b200.engine import memory_plan
from vllm_cpp_b200.parts.model import DecoderModel
from vllm_cpp_b200.weights.random_init import random_tensor

MIB = 1 << 20


def model_b(dtype=torch.bfloat16):
    _, spec = resolve_architecture(TINY_B, "")
    m = DecoderModel(spec, dtype, "cpu")
    m.load_params({n: random_tensor(n, ps.shape, ps.role, 0, 0.02, 0.02).to(m.placement(ps.role))
                   for n, ps in m.param_specs().items()})
    return m


def test_slices_and_pages_of_configuration_b():
    # hidden 96, 3 heads on 1 kv head of 32, intermediate 224, vocabulary 384, 3 layers, bfloat16
    cfg = EngineConfig(load_format="random", model_config=TINY_B, dtype="bfloat16", block_size=32, max_num_seqs=4,
                       max_model_len=512, max_num_batched_tokens=64, gpu_memory_utilization=90)
    m = model_b()
    # workspace of a step of 64 tokens, every piece rounded up to 256 bytes as the bump allocator does:
    #   the model's own: residual 64*96*4, delta 64*96*2, carried sums of squares 2*4*64*4, normed rows 4*96*2
    own = 24576 + 12288 + 2048 + 768
    #   a layer: two [64, 96] buffers and [4, 64] sums of squares, plus its greediest part, the feed-forward:
    #   activations 64*224*2 and the gate-and-up product 64*448*2 (attention: qkv 64*160*2 and twice 64*96*2)
    layer = 2 * 12288 + 1024 + max(28672 + 57344, 20480 + 2 * 12288)
    assert m.workspace_bytes(64, 4, 4) == own + layer == 151296
    total = 1 << 30
    budget = int(total * 0.9)
    expect = [
        ("step workspace (high-water mark)", 151552),                    # 151296 up to a multiple of 512
        ("logits [max_num_seqs, vocab] float32", 4 * 384 * 4),
        # ids, positions, request of token (3 x 64), starts (5 -> 8), contexts and slots (2 x 4), logit rows (64),
        # one block table of 4 x 16 entries, 64 Ki ints of room for the parts' work lists; 4 bytes each -> 512s
        ("step metadata (ids, positions, block tables)", 263680),
        ("sampler options and ids, two steps in flight", 2 * 3 * 512),
        ("top-k/top-p scratch [max_num_seqs, vocab]", 4 * 384 * 4),
        ("product scratch (partial tiles, tickets)", 148 * 2 * 256 * 128 * 4 + 16384 * 4),
        ("decode attention scratch (split merge)", 4 * 3 * 32 * 34 * 4 + 4096),
        # at most 256 captured steps of 8 launches a layer call and 4 around them, 8 KiB each
        ("captured decode steps (up to 256)", 256 * (8 * 3 + 4) * 8192),
        ("reserve for libraries and context", 384 * MIB),
    ]
    others = sum(b for _, b in expect)
    page = 3 * 2 * 1 * 32 * 32 * 2                                        # layers x (k, v) x kv heads x slots x head size x 2 bytes
    in_place = budget - others - 20 * page - 5                            # room for 20 pages and 5 bytes over
    p = memory_plan.plan_for_model(cfg, m, total, in_place, 512, sm_count=148)
    assert [r for r in p.rows if not r[0].startswith("(in place)")] == expect
    assert (p.bytes_per_page, p.num_pages, p.pages_wanted, p.workspace_bytes) == (page, 20, 64, 151552)
    weights = dict(p.rows)["(in place) weights"]
    # matrices in bfloat16: embedding and output 2 x 384 x 96, per layer qkv 160 x 96, o 96 x 96, gate and up
    # 448 x 96, down 96 x 224; in float32: per layer the bias of 160, two gains of 96; the final gain; per
    # layer the 16 divisors of the rotation
    assert weights == 2 * (2 * 384 * 96 + 3 * (160 * 96 + 96 * 96 + 448 * 96 + 96 * 224)) + 4 * (3 * (160 + 2 * 96 + 16) + 96)
    assert "pages: 20 x 12288 B" in p.table()
    # plenty of memory: never more pages than every request at full length needs
    assert memory_plan.plan_for_model(cfg, m, 64 << 30, 1 << 30, 512, 148).num_pages == 64
    # too little for one request of max_model_len: refused with the table
    with pytest.raises(ConfigError, match="16 are needed"):
        memory_plan.plan_for_model(cfg, m, total, in_place + 5 * page, 512, 148)


def test_float32_doubles_the_pages_and_the_compute_buffers():
    cfg = EngineConfig(load_format="random", model_config=TINY_B, dtype="float32", block_size=32, max_num_seqs=4,
                       max_model_len=512, max_num_batched_tokens=64)
    p = memory_plan.plan_for_model(cfg, model_b(torch.float32), 8 << 30, 1 << 30, 512, 148)
    assert p.bytes_per_page == 2 * 12288
    # residual and sums of squares stay float32; delta, normed rows and the layer's buffers double
    assert p.workspace_bytes == 24576 + 2 * 12288 + 2048 + 2 * 768 + 2 * (2 * 12288) + 1024 + 2 * (28672 + 57344)
