"""The command line: option names as the reference's, `info` without torch-side work."""

from __future__ import annotations

import json

import pytest

from inference_engine_b200 import cli
from tests import helpers as H
from tests.tiny_configs import TINY_B


def test_info_prints_the_shape(tmp_path, capsys):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert cli.main(["info", "--model", str(tmp_path), "--gpu-mem", "180"]) == 0
    out = capsys.readouterr().out
    assert "architecture        LlamaForCausalLM" in out
    assert "layers / hidden     3 / 96" in out
    assert "heads (q / kv)      3 / 1  (GQA groups: 3, head dim 32)" in out
    assert "On a 180 GiB GPU" in out and "KV tokens fit" in out


def test_generate_options_are_the_references():
    args = cli.build_parser().parse_args(["generate", "--model", "m", "--prompt", "hi"])
    assert (args.temperature, args.top_p, args.max_tokens, args.seed, args.device) == (0.7, 0.9, 256, None, "cuda")
    assert (args.max_num_seqs, args.max_num_batched_tokens, args.block_size, args.num_blocks) == (64, 4096, 16, None)
    assert args.gpu_memory_utilization == 0.9 and not args.no_chunked_prefill and not args.no_cuda_graphs
    with pytest.raises(SystemExit):
        cli.build_parser().parse_args(["serve", "--model", "m"])  # there is no server


@pytest.mark.gpu
def test_generate_runs_from_a_folder(tmp_path, capsys):
    folder = H.write_model_dir(tmp_path / "m", TINY_B, H.make_weights(TINY_B, seed=1))
    rc = cli.main(["generate", "--model", str(folder), "--prompt-ids", "5,17,3,99", "--temperature", "0",
                   "--max-tokens", "5", "--dtype", "float32", "--num-blocks", "16", "--block-size", "8",
                   "--max-num-seqs", "2", "--max-num-batched-tokens", "64"])
    assert rc == 0
    from tests import plain_llama

    want = plain_llama.greedy_generate(TINY_B, H.make_weights(TINY_B, seed=1), [5, 17, 3, 99], 5,
                                       stop_ids=(2, 3))
    captured = capsys.readouterr()
    assert captured.out.split() == [str(t) for t in want]
    assert "tokens/s" in captured.err
