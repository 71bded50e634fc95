"""The command line without a GPU: option names and defaults of the reference's
``generate`` (crates/vllm-cli/src/generate.rs:29-53) and engine options
(crates/vllm-cli/src/serve.rs:44-77), what is refused before anything is
loaded, and the random-weights command."""
import json

import pytest

from railgun_b200 import cli


def test_generate_options_and_defaults():
    ap = cli.make_parser()
    a = ap.parse_args(["generate", "-m", "dir", "-p", "some text"])
    assert (a.model, a.prompt, a.prompt_ids) == ("dir", "some text", None)
    assert (a.max_tokens, a.temperature, a.cuda_device, a.show_token_ids) == (128, 0.0, 0, False)
    assert (a.max_num_seqs, a.max_num_batched_tokens, a.block_size, a.num_gpu_blocks, a.max_model_len) == \
        (256, 4096, 16, 1000, 4096)
    a = ap.parse_args(["generate", "--model", "dir", "--prompt-ids", "1,2;3", "--max-tokens", "7", "--temperature",
                       "0.5", "--top-k", "40", "--top-p", "0.9", "--seed", "3", "--stop-token-ids", "2,9",
                       "--cuda-device", "1", "--show-token-ids", "--dtype", "f32"])
    assert (a.prompt_ids, a.max_tokens, a.temperature, a.top_k, a.top_p, a.seed) == ("1,2;3", 7, 0.5, 40, 0.9, 3)
    assert (a.stop_token_ids, a.cuda_device, a.show_token_ids, a.dtype) == ("2,9", 1, True, "f32")
    assert a.random_weights is None
    assert ap.parse_args(["generate", "-m", "dir", "--prompt-ids", "1", "--random-weights", "5"]).random_weights == 5


def test_log_level_comes_from_the_environment(monkeypatch):
    import logging
    import railgun_b200
    monkeypatch.setenv("RAILGUN_LOG", "error")
    railgun_b200.init_logging()
    assert railgun_b200.log.level == logging.ERROR
    monkeypatch.setenv("RAILGUN_LOG", "debug")
    railgun_b200.init_logging()
    assert railgun_b200.log.level == logging.DEBUG
    monkeypatch.delenv("RAILGUN_LOG")
    railgun_b200.init_logging()
    assert railgun_b200.log.level == logging.INFO              # the reference's default


@pytest.mark.parametrize("argv", [["generate", "-m", "dir"],                                  # no prompt at all
                                  ["generate", "-m", "dir", "-p", "text", "--prompt-ids", "1"],  # both kinds
                                  ["generate", "--prompt-ids", "1"],                           # no model
                                  ["serve", "-m", "dir"]])                                    # no server here
def test_generate_refuses_bad_command_lines(argv, capsys):
    with pytest.raises(SystemExit) as e:
        cli.make_parser().parse_args(argv)
    assert e.value.code == 2
    assert "usage:" in capsys.readouterr().err


def test_prompts_are_checked_before_anything_is_loaded(tmp_path, capsys):
    # a text prompt needs the folder's tokenizer.json
    assert cli.main(["generate", "-m", str(tmp_path), "-p", "hello"]) == 2
    assert "tokenizer.json does not exist" in capsys.readouterr().err
    (tmp_path / "tokenizer.json").write_text("{ not a tokenizer")
    assert cli.main(["generate", "-m", str(tmp_path), "-p", "hello"]) == 2
    assert "cannot read" in capsys.readouterr().err
    # prompts of ids need at least one id each
    assert cli.main(["generate", "-m", str(tmp_path), "--prompt-ids", " ; "]) == 2
    assert "at least one token" in capsys.readouterr().err


def test_random_weights_command_writes_a_model_folder(tmp_path, capsys):
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=32, num_attention_heads=2, num_key_value_heads=1,
               num_hidden_layers=1, intermediate_size=48, vocab_size=50, tie_word_embeddings=True)
    (tmp_path / "cfg.json").write_text(json.dumps(cfg))
    out = tmp_path / "model"
    assert cli.main(["random-weights", "--config", str(tmp_path / "cfg.json"), "--seed", "4", "--out", str(out)]) == 0
    assert json.loads(capsys.readouterr().out)["written"] == str(out)
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    again = tmp_path / "again"
    cli.main(["random-weights", "--config", str(tmp_path / "cfg.json"), "--seed", "4", "--out", str(again)])
    assert (out / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()      # seeded
    (tmp_path / "bad.json").write_text(json.dumps({"hidden_size": 8}))
    assert cli.main(["random-weights", "--config", str(tmp_path / "bad.json"), "--out", str(tmp_path / "x")]) == 2
