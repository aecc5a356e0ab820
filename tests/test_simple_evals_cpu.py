"""simple-evals style tasks: extraction, scoring, option shuffling, a run through the in-process engine."""
import json

import pytest

from maxtext_b200.eval import simple_evals as E


def test_number_and_letter_extraction():
  assert E.extract_number("so 3 + 4\nAnswer: 1,234.") == "1234" and E.extract_number("Answer: 7 apples") is None
  assert E.extract_number("Answer: 3\nbut then more text") is None and E.extract_number("x\n answer :  -12.5") == "-12.5"
  assert E.numbers_equal("18.0", "18") and not E.numbers_equal(None, "1") and not E.numbers_equal("abc", "1")
  assert E.extract_letter("I think Answer: B. wait, Answer: (C)") == "C" and E.extract_letter("none") is None
  assert E.f1_words("The cat sat.", "a cat sat") == 1.0 and E.f1_words("dog", "cat") == 0.0 and 0 < E.f1_words("big red cat", "red cat") < 1


def test_tasks_score_a_scripted_sampler(tmp_path):
  gsm = [{"question": "2+2?", "answer": "easy #### 4"}, {"question": "10*100?", "answer": "#### 1,000"}]
  replies = iter(["reasoning\nAnswer: 4", "hmm\nAnswer: 999"])
  r = E.run_task("gsm8k", gsm, lambda m: next(replies))
  assert r.n == 2 and r.score == 0.5 and r.samples[0].prompt[0]["content"].endswith("2+2?") and r.metrics["extracted"] == 1.0
  # gpqa: the options are shuffled per row, the target letter follows the correct answer
  row = {"Question": "Which?", "Correct Answer": "right", "Incorrect Answer 1": "w1", "Incorrect Answer 2": "w2", "Incorrect Answer 3": "w3"}
  seen = set()

  def pick_right(messages):
    text = messages[0]["content"]
    letter = [ln[0] for ln in text.splitlines() if ln[1:3] == ") " and ln.endswith("right")][0]
    seen.add(letter)
    return f"Answer: {letter}"
  g = E.run_task("gpqa", [row] * 12, pick_right, seed=1)
  assert g.score == 1.0 and len(seen) > 1
  m = E.run_task("mmlu", [{"question": "q", "choices": ["a", "b", "c", "d"], "answer": 2, "subject": "anatomy"}], lambda _: "Answer: C")
  assert m.score == 1.0 and m.samples[0].meta["subject"] == "anatomy"
  d = E.run_task("drop", [{"passage": "p", "question": "who?", "answers": ["John Smith", "Smith"]}], lambda _: "thinking\nAnswer: john smith")
  assert d.score == 1.0
  a = E.run_task("aime", [{"problem": "p", "answer": "073"}], lambda _: "Answer: 73")
  assert a.score == 1.0
  with pytest.raises(KeyError):
    E.run_task("nope", [], lambda _: "")
  path = E.write_report(r, str(tmp_path))
  assert json.load(open(path))["samples"][1]["extracted"] == "999"
  f = tmp_path / "rows.jsonl"
  f.write_text("\n".join(json.dumps(x) for x in gsm))
  assert E.load_rows(str(f), 1) == gsm[:1]


def test_engine_sampler_answers_through_the_chat_template():
  from helpers import tiny_config
  from maxtext_b200.eval.runner import LocalBackend
  from maxtext_b200.input_pipeline.tokenizer import ByteTokenizer
  cfg = tiny_config("llama3-8b", ["vocab_size=300", "max_target_length=400", "max_prefill_predict_length=360", "per_device_batch_size=2"])
  s = E.EngineSampler(cfg, backend=LocalBackend(cfg, tokenizer=ByteTokenizer(), slots=2), max_new_tokens=4)
  r = E.run_task("gsm8k", [{"question": "1+1?", "answer": "#### 2"}], s)
  assert r.n == 1 and isinstance(r.samples[0].response, str) and 0.0 <= r.score <= 1.0
