"""Text prompts and chat: the tokenizer wrapper, the chat template, the tokenizer's end-of-sequence
id among the ids that end a request, LLM.chat() and the command line's --chat.  No GPU: the kernels
are replaced by their plain restatements."""

import json

import pytest

import kernel_refs
from tiny_configs import TINY_A

from emberserve_b200.engine.runner import ModelRunner

tokenizers = pytest.importorskip("tokenizers")

WORDS = ["<unk>", "<|im_start|>", "<|im_end|>", "<|endoftext|>", "user", "assistant", "system", "hello",
         "world", "how", "are", "you", "fine", "\n"]


def write_tokenizer(folder, template: str | None = "default", eos: str | dict | None = "<|im_end|>"):
    """A word-level tokenizer over a handful of words; special tokens are matched as written."""
    from tokenizers import Tokenizer, models, pre_tokenizers

    vocab = {w: i for i, w in enumerate(WORDS)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split(" ", behavior="removed")
    tok.add_special_tokens(["<|im_start|>", "<|im_end|>", "<|endoftext|>"])
    tok.save(str(folder / "tokenizer.json"))
    cfg = {}
    if eos is not None:
        cfg["eos_token"] = eos
    if template == "default":
        cfg["chat_template"] = (
            "{% for m in messages %}{{ '<|im_start|> ' + m['role'] + ' ' + m['content'] + ' <|im_end|> ' }}"
            "{% endfor %}{% if add_generation_prompt %}{{ '<|im_start|> assistant' }}{% endif %}")
    elif template is not None:
        cfg["chat_template"] = template
    (folder / "tokenizer_config.json").write_text(json.dumps(cfg))


def ids(*words):
    return [WORDS.index(w) for w in words]


def test_wrapper_encodes_decodes_and_reads_eos(tmp_path):
    from emberserve_b200.tokenizer import Tokenizer, has_tokenizer, load_tokenizer

    assert not has_tokenizer(tmp_path) and load_tokenizer(tmp_path) is None
    write_tokenizer(tmp_path, eos={"content": "<|im_end|>", "lstrip": False})
    assert has_tokenizer(tmp_path)
    tok = Tokenizer(tmp_path)
    assert tok.encode("hello world") == ids("hello", "world")
    assert tok.decode(ids("how", "are", "you")) == "how are you"
    assert tok.decode_batch([ids("hello"), ids("fine", "you")]) == ["hello", "fine you"]
    assert tok.eos_token_id == WORDS.index("<|im_end|>")


def test_chat_template_of_the_folder_is_rendered(tmp_path):
    from emberserve_b200.tokenizer import Tokenizer

    write_tokenizer(tmp_path)
    tok = Tokenizer(tmp_path)
    msgs = [{"role": "system", "content": "hello"}, {"role": "user", "content": "how are you"}]
    want = ids("<|im_start|>", "system", "hello", "<|im_end|>", "<|im_start|>", "user", "how", "are", "you",
               "<|im_end|>", "<|im_start|>", "assistant")
    assert tok.apply_chat_template(msgs) == want
    assert tok.apply_chat_template(msgs, add_generation_prompt=False) == want[:-2]
    with pytest.raises(ValueError, match="role"):
        tok.apply_chat_template([{"content": "x"}])


def test_template_file_wins_and_templates_may_refuse(tmp_path):
    from emberserve_b200.tokenizer import Tokenizer

    write_tokenizer(tmp_path, template="{{ raise_exception('no system turn') }}")
    with pytest.raises(ValueError, match="no system turn"):
        Tokenizer(tmp_path).apply_chat_template([{"role": "user", "content": "hello"}])
    (tmp_path / "chat_template.jinja").write_text("{{ bos_token }}{{ messages[0]['content'] }} {{ eos_token }}")
    tok = Tokenizer(tmp_path)
    assert tok.apply_chat_template([{"role": "user", "content": "fine"}]) == ids("fine", "<|im_end|>")


def test_without_a_template_the_layout_is_chatml(tmp_path):
    from emberserve_b200.tokenizer import Tokenizer, chatml

    write_tokenizer(tmp_path, template=None)
    text = Tokenizer(tmp_path).render_chat([{"role": "user", "content": "hello"}])
    assert text == "<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n"
    assert chatml([{"role": "user", "content": "a"}], add_generation_prompt=False) == "<|im_start|>user\na<|im_end|>\n"


@pytest.fixture()
def model_folder(tmp_path, monkeypatch):
    from emberserve_b200.weights.loader import write_random_model

    kernel_refs.install(monkeypatch)
    monkeypatch.setattr(ModelRunner, "_require_cuda", False)  # host logic only, as in host_harness
    folder = write_random_model(TINY_A, tmp_path / "model", seed=3)
    write_tokenizer(folder)
    return folder


def test_engine_ends_on_the_tokenizers_eos_and_chat_goes_through_the_template(model_folder):
    from emberserve_b200 import LLM, SamplingParams

    llm = LLM(model_folder, dtype="float32", device="cpu", block_size=4, num_gpu_blocks=64, max_model_len=64,
              enable_cuda_graphs=False)
    assert WORDS.index("<|im_end|>") in llm.engine.eos_token_ids
    assert set(TINY_A.eos_token_ids) <= llm.engine.eos_token_ids
    conv = [{"role": "user", "content": "how are you"}]
    res = llm.chat([conv], SamplingParams.greedy(4, ignore_eos=True))[0]
    assert res.prompt_token_ids == llm.engine.tokenizer.apply_chat_template(conv)
    same = llm.generate([res.prompt_token_ids], SamplingParams.greedy(4, ignore_eos=True))[0]
    assert same.output_token_ids == res.output_token_ids
    assert res.text == llm.engine.tokenizer.decode(res.output_token_ids)
    text = llm.generate(["hello world"], SamplingParams.greedy(2, ignore_eos=True))[0]
    assert text.prompt_token_ids == ids("hello", "world")
    # the text of a request that has ended can be asked for once, that of a live one at any time
    assert llm.engine.output_text("req-0") == text.text
    assert llm.engine.output_text("req-0") == ""
    llm.engine.add_request("live", "how are you", SamplingParams.greedy(6, ignore_eos=True))
    pieces = []
    while llm.engine.has_unfinished_requests():
        for out in llm.engine.step():
            pieces.append(out.text_delta)
            if not out.finished:
                assert llm.engine.output_text("live") == "".join(pieces)
    assert llm.engine.output_text("live") == "".join(pieces)


def test_chat_needs_a_tokenizer(tmp_path, monkeypatch):
    from emberserve_b200 import LLM
    from emberserve_b200.weights.loader import write_random_model

    kernel_refs.install(monkeypatch)
    monkeypatch.setattr(ModelRunner, "_require_cuda", False)
    folder = write_random_model(TINY_A, tmp_path / "bare", seed=3)
    llm = LLM(folder, dtype="float32", device="cpu", block_size=4, num_gpu_blocks=32, max_model_len=64,
              enable_cuda_graphs=False)
    with pytest.raises(ValueError, match="tokenizer"):
        llm.chat([[{"role": "user", "content": "hello"}]])


def test_command_line_chat(model_folder, capsys):
    from emberserve_b200.cli import main

    common = ["generate", "--model", str(model_folder), "--dtype", "float32", "--device", "cpu", "--block-size", "4",
              "--num-blocks", "64", "--max-model-len", "64", "--no-cuda-graphs", "--max-tokens", "3"]
    assert main(common + ["--prompt", "how are you", "--chat"]) == 0
    chat_out = capsys.readouterr().out
    assert main(common + ["--prompt", "how are you"]) == 0
    plain_out = capsys.readouterr().out
    assert chat_out.strip() and plain_out.strip()
    with pytest.raises(SystemExit):
        main(common + ["--prompt-ids", "1,2,3", "--chat"])
