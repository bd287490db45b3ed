"""Benchmark drivers on CPU: judge client (retry, refusal), answer parsers, metrics, resumable logs,
the image-judging driver and the interleave / understanding scorers against a stand-in judge served over HTTP."""
import json
import threading
from http.server import BaseHTTPRequestHandler, HTTPServer
from pathlib import Path

import pytest

from evaluation.common import metrics
from evaluation.common.judge import (JudgeClient, JudgeError, ResultLog, merge_shards, parse_choice, parse_json_block,
                                     parse_score, parse_yes_no, run_parallel)


class _Judge(BaseHTTPRequestHandler):
    fail_first = 0          # answer 503 this many times before working
    seen = []

    def log_message(self, *a):
        pass

    def do_POST(self):
        body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
        cls = type(self)
        if cls.fail_first > 0:
            cls.fail_first -= 1
            self.send_response(503)
            self.end_headers()
            return
        user = body["messages"][-1]["content"]
        text = user if isinstance(user, str) else user[0]["text"]
        n_img = 0 if isinstance(user, str) else sum(1 for p in user if p["type"] == "image_url")
        cls.seen.append((text, n_img))
        if "forbidden" in text:
            self.send_response(400)
            self.end_headers()
            return
        if text.startswith("Transcribe"):
            ans = "GRAND  Opening, today!"
        elif text.startswith("Prompt:") or text.startswith("Task:"):
            ans = "score: 7 - mostly right"
        elif "Answer with the option letter" in text:
            ans = "The shape repeats, so Answer: B"
        elif "single word" in text:
            ans = "42%"
        else:
            ans = "Yes, it is there." if "cat" in text else "No."
        out = json.dumps({"choices": [{"message": {"role": "assistant", "content": ans}}]}).encode()
        self.send_response(200)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(out)))
        self.end_headers()
        self.wfile.write(out)


@pytest.fixture()
def judge_url():
    _Judge.fail_first, _Judge.seen = 0, []
    srv = HTTPServer(("127.0.0.1", 0), _Judge)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    yield f"http://127.0.0.1:{srv.server_address[1]}"
    srv.shutdown()
    t.join(timeout=5)


def _png(path, size=(32, 32)):
    from PIL import Image
    path.parent.mkdir(parents=True, exist_ok=True)
    Image.new("RGB", size, (200, 10, 10)).save(path)


def test_parsers():
    assert parse_yes_no("Yes, clearly.") is True and parse_yes_no(" no - absent") is False and parse_yes_no("maybe") is None
    assert parse_score("score: 7 because") == 7 and parse_score("I give 8/10") == 8 and parse_score("12") is None
    assert parse_score('{"score": 6.5}') == 6.5
    assert parse_json_block('sure:\n```json\n{"a": 1}\n```') == {"a": 1} and parse_json_block('x {"b": {"c": 2}} y') == {"b": {"c": 2}}
    assert parse_choice("so the Answer: (C).") == "C" and parse_choice("I think it is **B**") == "B"
    assert parse_choice("nothing here", "ABCD") is None


def test_metrics():
    assert metrics.edit_distance("kitten", "sitting") == 3
    assert metrics.word_accuracy("grand opening TODAY", ["Grand Opening", "today!"]) == 1.0
    assert metrics.word_accuracy("grand", ["grand grand"]) == 0.5
    assert metrics.normalized_edit_distance("abc", "abc") == 1.0 and metrics.normalized_edit_distance("", "abcd") == 0.0
    s = metrics.checklist_scores([{"dimension": "text", "checks": [True, False]}, {"dimension": "layout", "checks": [True, None, True, True]}])
    assert s["dim/text"] == 0.5 and s["dim/layout"] == 0.75 and s["overall"] == 0.625
    assert metrics.relaxed_match("It is 41.0", ["42"]) == 0.0 and metrics.relaxed_match("41", ["42"]) == 1.0
    assert metrics.relaxed_match("the answer is a red fox.", ["red fox"]) == 1.0
    assert metrics.anls("invoice 1234", ["Invoice 1234"]) == 1.0 and metrics.anls("zzz", ["invoice"]) == 0.0
    acc = metrics.accuracy_by_category([{"category": "a", "correct": 1.0}, {"category": "a", "correct": 0.0}, {"category": "b", "correct": 1.0}, {"correct": None}])
    assert acc["cat/a"] == 0.5 and acc["accuracy"] == pytest.approx(2 / 3) and acc["n"] == 3


def test_client_retries_then_reports(judge_url, tmp_path):
    naps = []
    c = JudgeClient(judge_url, model="judge", max_retries=3, sleep=naps.append)
    _Judge.fail_first = 2
    assert c.ask("is there a cat?") == "Yes, it is there."
    assert c.retries == 2 and naps == [1.0, 2.0]
    with pytest.raises(JudgeError):
        c.ask("forbidden question")                       # a 4xx answer is not retried
    _Judge.fail_first = 10
    with pytest.raises(JudgeError):
        JudgeClient(judge_url, model="judge", max_retries=1, sleep=naps.append).ask("is there a cat?")
    with pytest.raises(ValueError):
        JudgeClient("", model="")


def test_resumable_log_and_shards(tmp_path):
    log = ResultLog(tmp_path / "r.jsonl")
    calls = []

    def fn(it):
        calls.append(it["id"])
        if it["id"] == "2":
            raise RuntimeError("broken sample")
        return {"v": int(it["id"]) * 2}

    run_parallel([{"id": str(i)} for i in range(4)], fn, log, workers=2)
    assert sorted(calls) == ["0", "1", "2", "3"] and "error" in log.done["2"]
    with open(tmp_path / "r.jsonl", "a") as f:
        f.write('{"id": "9", "v"')                          # a line cut off by a crash
    log2 = ResultLog(tmp_path / "r.jsonl")
    run_parallel([{"id": str(i)} for i in range(6)], fn, log2, workers=2)
    assert sorted(calls) == ["0", "1", "2", "3", "4", "5"]    # only the new ones ran
    (tmp_path / "a.jsonl").write_text('{"id": "1", "x": 1}\n')
    (tmp_path / "b.jsonl").write_text('{"id": "1", "x": 2}\n{"id": "10", "x": 3}\n')
    assert merge_shards([tmp_path / "a.jsonl", tmp_path / "b.jsonl"], tmp_path / "m.jsonl") == 2
    assert [json.loads(l)["x"] for l in (tmp_path / "m.jsonl").read_text().splitlines()] == [2, 3]


def test_image_judging_driver(judge_url, tmp_path, monkeypatch):
    from evaluation.gen import judge_images
    run = tmp_path / "run"
    for i in range(2):
        for k in range(2):
            _png(run / f"{i:05d}" / "samples" / f"{k:04d}.png")
    recs = [{"index": 0, "prompt": "a cat on a sofa", "samples": 2, "dimension": "object", "questions": ["is there a cat?", "is there a dog?"],
             "target_texts": ["Grand Opening", "Today"]},
            {"index": 1, "prompt": "a dog", "samples": 2, "dimension": "attribute", "questions": ["is the cat red?"], "target_texts": ["Closed"]}]
    (run / "metadata.rank0.jsonl").write_text("\n".join(json.dumps(r) for r in recs))
    monkeypatch.setenv("JUDGE_API_BASE", judge_url)
    monkeypatch.setenv("JUDGE_MODEL", "judge")
    s = judge_images.main(["--run", str(run), "--mode", "checklist", "--workers", "2"])
    assert s["n"] == 4 and s["dim/object"] == 0.5 and s["dim/attribute"] == 1.0 and s["errors"] == 0
    assert all(n == 1 for _, n in _Judge.seen)                 # every question carried its picture
    before = len(_Judge.seen)
    judge_images.main(["--run", str(run), "--mode", "checklist"])
    assert len(_Judge.seen) == before                          # resumed: nothing asked twice
    s = judge_images.main(["--run", str(run), "--mode", "text"])
    assert s["word_accuracy"] == pytest.approx((1.0 + 0.0) / 2) and s["all_words_right"] == 0.5
    s = judge_images.main(["--run", str(run), "--mode", "rating"])
    assert s["overall"] == 7.0 and json.loads((run / "scores_rating.json").read_text())["n"] == 4


def test_interleave_and_understanding_scoring(judge_url, tmp_path, monkeypatch):
    from evaluation.interleave import infer, score
    from evaluation.understanding import run_vqa
    data = tmp_path / "data"
    _png(data / "q.png")
    qs = [{"id": "a", "question": "which comes next?", "images": ["q.png"], "options": ["circle", "square", "star"], "answer": "B", "category": "pattern"},
          {"id": "b", "question": "which comes next?", "options": ["circle", "square"], "answer": "circle", "category": "pattern"},
          {"id": "c", "question": "how many?", "answer": "3", "category": "count"}]
    (data / "q.jsonl").write_text("\n".join(json.dumps(q) for q in qs))

    def fake_model(question, paths):
        return ("thinking...\nAnswer: B" if "option letter" in question else "there are\n3"), [b"\x89PNG fake"]

    out = tmp_path / "run"
    recs = [dict(q, _root=str(data)) for q in qs]
    infer.run(recs[:2], fake_model, out, ResultLog(out / "predictions_000.jsonl"))
    infer.run(recs[2:], fake_model, out, ResultLog(out / "predictions_001.jsonl"))
    assert (out / "images" / "a_0.png").exists()
    s = score.main(["--run", str(out)])
    assert s["cat/pattern"] == 0.5 and s["cat/count"] == 1.0 and s["n"] == 3     # "circle" is option A, the model said B
    monkeypatch.setenv("JUDGE_API_BASE", judge_url)
    monkeypatch.setenv("JUDGE_MODEL", "judge")
    (out / "images" / "a_0.png").unlink()
    _png(out / "images" / "a_0.png")
    for n in ("b_0.png", "c_0.png"):
        _png(out / "images" / n)
    s = score.main(["--run", str(out), "--judge", "--workers", "2"])
    assert s["overall"] == 7.0 and s["n"] == 3
    vq = [{"id": "1", "question": "which?", "images": ["q.png"], "options": ["x", "y"], "answer": "B"},
          {"id": "2", "question": "what share?", "images": ["q.png"], "answer": ["41"], "category": "chart"},
          {"id": "3", "question": "what share?", "answer": "50", "metric": "exact"}]
    (data / "v.jsonl").write_text("\n".join(json.dumps(q) for q in vq))
    s = run_vqa.main(["--data", str(data / "v.jsonl"), "--out", str(tmp_path / "vqa"), "--base_url", judge_url, "--workers", "2"])
    assert s["accuracy"] == pytest.approx(2 / 3) and s["cat/chart"] == 1.0 and s["errors"] == 0


# ---------------------------------------------------------------------------
# per-benchmark scoring rules
# ---------------------------------------------------------------------------
def test_benchmark_rules():
    from evaluation.benchmarks import (babyvision_summary, bizgeneval_summary, cvtg_summary, igenbench_summary,
                                       longtext_summary, opening_summary, realunify_summary, tiif_summary,
                                       unimmmu_summary)
    biz = bizgeneval_summary([
        {"checks": [True, False, True, None], "easy_qidxs": [1, 2], "hard_qidxs": [3, 4], "domain": "poster", "dimension": "layout"},
        {"checks": [True, True], "easy_qidxs": [1], "hard_qidxs": [2], "domain": "chart", "dimension": "layout"}])
    assert abs(biz["overall_accuracy"] - (0.5 + 1.0) / 2) < 1e-9
    assert abs(biz["overall_error_score"] - (0.8 + 1.0) / 2) < 1e-9                 # 1 - 0.1 * 2 failures
    assert abs(biz["easy_error_score"] - (0.8 + 1.0) / 2) < 1e-9 and biz["by_dimension"]["layout"]["count"] == 2
    ig = igenbench_summary([{"checks": [True, True], "question_types": ["value", "label"]},
                            {"checks": [True, False, False], "question_types": ["value", "value", "label"]}])
    assert abs(ig["score"] - (1.0 + 1 / 3) / 2) < 1e-9 and abs(ig["q_acc"] - 3 / 5) < 1e-9 and ig["i_acc_strict"] == 0.5
    assert abs(ig["question_type_acc"]["value"] - 2 / 3) < 1e-9
    lt = longtext_summary([{"target_texts": "Hello, big World!", "read_text": "hello world world"},
                           {"target_texts": ["one two"], "read_text": ""}])
    assert abs(lt["score"] - 2 / 5) < 1e-9
    zh = longtext_summary([{"target_texts": "你好，世界", "read_text": "你 好 世"}], mode="zh")
    assert abs(zh["score"] - 3 / 4) < 1e-9
    cv = cvtg_summary([{"prompt": "a sign reading 'open late' and a cup saying 'joe'", "read_text": "OPEN lite joe", "area": 2}])
    assert abs(cv["word_accuracy"] - 2 / 3) < 1e-9 and 0.8 < cv["ned"] < 1.0 and cv["by_area"]["2"]["count"] == 1
    tf = tiif_summary([{"gt_answers": ["yes", "no"], "model_pred": ["Yes", "yes"], "attribute": "color", "type": "short"}])
    assert tf["cells"]["color/short"]["accuracy"] == 0.5
    ru = realunify_summary([{"model_response": "I think <answer>b</answer>", "answer": "B", "task_type": "gen"},
                            {"response": ["C."], "answer": "A", "task_type": "gen"}])
    assert ru["by_task"]["gen"]["acc"] == 0.5
    um = unimmmu_summary([{"task": "jigsaw", "correct": True}, {"task": "maze", "response": "D", "answer": "D"},
                          {"task": "maze", "response": "A", "answer": "D"}])
    assert um["by_task"]["maze"]["acc"] == 0.5 and abs(um["task_mean_acc"] - 0.75) < 1e-9
    bv = babyvision_summary([{"LLMJudgeResult": True, "Type": "Visual Tracking", "Subtype": "maze"},
                             {"LLMJudgeResult": False, "Type": "Visual Tracking", "Subtype": "lines"}])
    assert bv["overall_accuracy"] == 0.5 and "2Visual Tracking/maze" in bv["by_subtype"]
    op = opening_summary([{"model": {"id": "m1", "name": "ours"}, "score": {"scores": {"quality": 8, "coherence": 6}}},
                          {"model": {"id": "m1", "name": "ours"}, "score": None},
                          {"model": {"id": "m2", "name": "other"}, "score": {"quality": 5, "coherence": 5}}])
    assert op["dropped"] == 1 and op["ranking"] == ["ours", "other"] and op["models"]["ours"]["overall"] == 7.0


def test_benchmark_score_cli(tmp_path, capsys):
    import json
    from evaluation.benchmarks.score import main
    f = tmp_path / "r.jsonl"
    f.write_text(json.dumps({"checks": [True, False], "domain": "d", "dimension": "x"}) + "\n")
    assert main(["--benchmark", "bizgeneval", "--records", str(f), "--out", str(tmp_path / "s.json")]) == 0
    assert json.loads((tmp_path / "s.json").read_text())["overall_accuracy"] == 0.5


# ---------------------------------------------------------------------------------------------------------------
# per-benchmark generation / judging pipelines (stand-in painter and judge)
# ---------------------------------------------------------------------------------------------------------------
class _FakeJudge:
    """Answers by the protocol of the question it is asked."""
    model = "fake-judge"

    def __init__(self):
        self.calls = 0

    def ask(self, question, images=(), system=None, temperature=0.0, max_tokens=1024):
        self.calls += 1
        assert images and Path(images[0]).exists()
        if "Statements:" in question:                                  # BizGenEval checklist, Python literals on purpose
            n = question.count("\n") - 1
            return "```json\n{" + ", ".join(f'"{i}": {{"result": {"True" if i % 2 else "False"}, "reason": "r"}}'
                                            for i in range(1, n + 1)) + "}\n```"
        if "infographic" in question:
            return '{"analysis": "seen", "answer": "%d"}' % (0 if "pie" in question else 1)
        if "Recognize the text" in question:
            return "FRESH BREWS every morning\nNo text recognized."
        if "yes-or-no" in question:
            qs = question.split("Questions:\n")[1].split("\nOne line")[0].splitlines()
            return "\n".join(("yes, visible" if "cat" in q else "no, absent") for q in qs)
        raise AssertionError(question)


def _painter(log):
    from PIL import Image

    def draw(prompt, size, a):
        log.append((prompt, size))
        return [Image.new("RGB", (size[0] // 16, size[1] // 16), (10, 20, 30)) for _ in range(a.batch_size)]
    return draw


def test_bizgeneval_pipeline(tmp_path):
    from evaluation.gen import run_benchmark as rb
    data = tmp_path / "test.jsonl"
    rows = [{"id": 7, "domain": "webpage", "dimension": "layout", "aspect_ratio": "4:3", "prompt": "a page",
             "questions": ["q1", "q2", "q3"], "easy_qidxs": [1], "hard_qidxs": [2, 3]},
            {"id": 8, "domain": "poster", "dimension": "text", "aspect_ratio": "2400x3000", "prompt": "a poster",
             "questions": ["q1"], "easy_qidxs": [1], "hard_qidxs": []}]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    drawn = []
    out = rb.main(["generate", "bizgeneval", "--output-dir", str(tmp_path / "img"), "--data-path", str(data),
                   "--random_init", "tiny-mot"], draw=_painter(drawn))
    assert out == {"prompts": 2, "generated": 2, "skipped": 0}
    assert [s for _, s in drawn] == [(2048, 1536), (1632, 2048)]                 # long side 2048, multiples of 32
    assert (tmp_path / "img" / "0000.png").exists() and (tmp_path / "img" / "0001.png").exists()
    again = rb.main(["generate", "bizgeneval", "--output_dir", str(tmp_path / "img"), "--data_path", str(data)], draw=_painter(drawn))
    assert again["generated"] == 0 and len(drawn) == 2                            # resumes
    judge = _FakeJudge()
    s = rb.main(["evaluate", "bizgeneval", "--image-dir", str(tmp_path / "img"), "--output-dir", str(tmp_path / "ev"),
                 "--data-path", str(data)], client=judge)
    assert judge.calls == 2 and s["judged"] == 2 and s["missing_images"] == 0
    # item 0: statements 1,3 true, 2 false -> accuracy 2/3, one error -> 0.9; item 1: all true
    assert s["overall_accuracy"] == pytest.approx((2 / 3 + 1) / 2) and s["overall_error_score"] == pytest.approx(0.95)
    assert s["hard_error_score"] == pytest.approx((0.8 + 0.0) / 2) and s["easy_error_score"] == pytest.approx(1.0)
    assert json.loads((tmp_path / "ev" / "bizgeneval_summary.json").read_text())["benchmark"] == "bizgeneval"
    rb.main(["evaluate", "bizgeneval", "--image_dir", str(tmp_path / "img"), "--output_dir", str(tmp_path / "ev"),
             "--data_path", str(data)], client=judge)
    assert judge.calls == 2                                                       # judged items are not asked again


def test_igenbench_and_longtext_pipelines(tmp_path):
    from evaluation.gen import run_benchmark as rb
    d = tmp_path / "igen"
    d.mkdir()
    (d / "3.json").write_text(json.dumps({"id": 3, "t2i_prompt": "bars", "chart_type": "bar", "evaluation": [
        {"question": "Is there a bar chart?", "question_type": "chart"}, {"question": "Is there a pie?", "question_type": "chart"},
        {"question": "Is the title right?", "question_type": "text"}, {"question": " "}]}))
    (d / "notes.json").write_text("{}")
    drawn = []
    rb.main(["generate", "igenbench", "--output_dir", str(tmp_path / "img"), "--data_dir", str(d)], draw=_painter(drawn))
    assert drawn == [("bars", (2048, 2048))] and (tmp_path / "img" / "0003.png").exists()
    s = rb.main(["evaluate", "igenbench", "--image_dir", str(tmp_path / "img"), "--output_dir", str(tmp_path / "ev"),
                 "--data_dir", str(d)], client=_FakeJudge())
    assert s["q_acc"] == pytest.approx(2 / 3) and s["i_acc_strict"] == 0.0
    assert s["question_type_acc"] == {"chart": 0.5, "text": 1.0}

    lt = tmp_path / "lt.jsonl"
    lt.write_text(json.dumps({"prompt_id": 5, "prompt": "a sign", "text": ["FRESH BREWS,", "EVERY MORNING, EVERY DAY"],
                              "category": "sign", "length": "short"}) + "\n")
    rb.main(["generate", "longtext", "--output_dir", str(tmp_path / "lti"), "--data_path", str(lt), "--aspect_ratio", "16:9"],
            draw=_painter(drawn))
    assert drawn[-1] == ("a sign", (2720, 1536))
    s = rb.main(["evaluate", "longtext", "--image_dir", str(tmp_path / "lti"), "--output_dir", str(tmp_path / "lte"),
                 "--data_path", str(lt)], client=_FakeJudge())
    assert s["benchmark"] == "longtext_en" and s["score"] == pytest.approx(4 / 6)   # fresh brews every morning | every day
    assert s["by_length"]["short"]["count"] == 1


def test_cvtg_and_tiif_pipelines(tmp_path, monkeypatch):
    from evaluation.gen import run_benchmark as rb
    root = tmp_path / "cvtg"
    (root / "CVTG").mkdir(parents=True)
    (root / "CVTG" / "2_combined.json").write_text(json.dumps({"a1": "a cafe sign 'fresh brews' and a note 'every night'",
                                                               "a2": "skip"}))
    drawn = []
    rb.main(["generate", "cvtg", "--output_dir", str(tmp_path / "ci"), "--benchmark_root", str(root), "--subsets", "CVTG",
             "--areas", "2", "--target_keys", "a1", "--save_size", "1024"], draw=_painter(drawn))
    a = rb.parser().parse_args(["generate", "cvtg", "--output_dir", "x"])
    assert a.cfg_scale == 7.0 and a.timestep_shift == 1.0                           # the benchmark's own sampling defaults
    from PIL import Image
    assert Image.open(tmp_path / "ci" / "CVTG" / "2" / "a1.png").size == (64, 64) and len(drawn) == 1   # the painter draws 1/16 scale; saved at half of that
    s = rb.main(["evaluate", "cvtg", "--result_dir", str(tmp_path / "ci"), "--output_dir", str(tmp_path / "ce"),
                 "--benchmark_root", str(root), "--subsets", "CVTG", "--areas", "2", "--target_keys", "a1"], client=_FakeJudge())
    assert s["judged"] == 1 and 0.0 < s["word_accuracy"] < 1.0

    td = tmp_path / "tiif"
    td.mkdir()
    (td / "color.jsonl").write_text("\n".join(json.dumps(r) for r in [
        {"type": "color", "short_description": "a red cat", "long_description": "a very red cat on a mat",
         "yn_question_list": ["Is there a cat?", "Is there a dog?"], "yn_answer_list": ["yes", "no"]},
        {"type": "color", "short_description": "a blue dog", "long_description": "a blue dog outside",
         "yn_question_list": ["Is there a cat?"], "yn_answer_list": ["no"]}]))
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("WORLD_SIZE", "2")
    r1 = rb.main(["generate", "tiif", "--output_dir", str(tmp_path / "ti"), "--input_folder", str(td), "--batch_size", "2",
                  "--rows", "1", "--cols", "2"], draw=_painter(drawn))
    monkeypatch.setenv("RANK", "0")
    r0 = rb.main(["generate", "tiif", "--output_dir", str(tmp_path / "ti"), "--input_folder", str(td), "--batch_size", "2",
                  "--rows", "1", "--cols", "2"], draw=_painter(drawn))
    assert r0["generated"] == 2 and r1["generated"] == 2                            # ranks split the four pictures
    grid = Image.open(tmp_path / "ti" / "color" / "sensenova-u1" / "long_description" / "1.png")
    assert grid.size == (2 * 64 + 2, 64)
    monkeypatch.delenv("RANK")
    monkeypatch.delenv("WORLD_SIZE")
    s = rb.main(["evaluate", "tiif", "--image_dir", str(tmp_path / "ti"), "--output_dir", str(tmp_path / "te"),
                 "--jsonl_dir", str(td)], client=_FakeJudge())
    assert s["judged"] == 4 and s["failed"] == 0
    with pytest.raises(SystemExit):
        rb.main(["generate", "tiif", "--output_dir", str(tmp_path / "ti"), "--input_folder", str(td), "--batch_size", "4"])


# ---------------------------------------------------------------------------------------------------------------
# interleaved benchmarks (stand-in engine and judge)
# ---------------------------------------------------------------------------------------------------------------
class _FakeEngine:
    def __init__(self):
        self.calls = []

    def _pic(self, size, colour=(200, 10, 10)):
        from PIL import Image
        return Image.new("RGB", (size[0] // 16, size[1] // 16), colour)

    def t2i(self, prompt, size):
        self.calls.append(("t2i", prompt, size))
        return self._pic(size)

    def edit(self, prompt, images, size):
        self.calls.append(("edit", prompt, size))
        return self._pic(size, (10, 200, 10))

    def ask(self, question, images=(), max_new_tokens=512, **gen):
        self.calls.append(("ask", question, len(images)))
        if "<answer>" in question:
            return "<think>count them</think>\n<answer>B</answer>" if "Choices" in question else "It is 7, so the answer is 7"
        if not images:
            return "a refined prompt"
        return "B: the left one"

    def interleave(self, prompt, images, size, system=None, think=True, max_new_tokens=4096, max_images=None):
        self.calls.append(("interleave", prompt, size, think, max_images))
        n = max_images or 1
        text = "<think>draft [image]</think>" + " [image] ".join(f"step {k}" for k in range(n)) + (" [image]" if n else "")
        if max_images is None:
            text = "<think>sketch [image] ok</think>C"
        return text, [self._pic(size) for _ in range(n)]


class _FakeTextJudge:
    model = "fake"

    def __init__(self):
        self.calls = 0

    def ask(self, question, images=(), system=None, temperature=0.0, max_tokens=1024):
        self.calls += 1
        if "only reply yes or no" in question:
            return "Yes." if "red" in question else "No"
        if "Extracted Answer" in question:
            a = question.split("Extracted Answer: ")[1].split("\n")[0]
            gt = question.split("Ground Truth: ")[1].split("\n")[0]
            return json.dumps({"is_correct": a.strip() == gt.strip()})
        if "INPUT:" in question:
            assert len(images) == 3
            from evaluation.interleave.suites import OPENING_CRITERIA
            return "```json\n" + json.dumps({c: {"Score": 6 + (k % 2), "Justification": "j"} for k, c in enumerate(OPENING_CRITERIA)}) + "\n```"
        raise AssertionError(question)


def test_realunify_pipelines(tmp_path, monkeypatch):
    from evaluation.interleave import run_benchmark as rb
    _png(tmp_path / "in.png", (640, 480))
    data = tmp_path / "geu.jsonl"
    rows = [{"hash_uid": f"u{i}", "task_type": "mental_tracking", "input_image": "in.png", "edit_prompt": "move it",
             "evaluation_prompt": "Which one? A, B, C or D.", "answer": a, "index": i} for i, a in enumerate("BC")]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    eng = _FakeEngine()
    r = rb.main(["infer", "realunify", "--data-path", str(data), "--output-dir", str(tmp_path / "step"), "--inference-mode", "step",
                 "--min_pixels", str(512 * 512), "--max_pixels", str(1024 * 1024)], engine=eng)
    assert r["new"] == 2 and r["failed"] == 0
    assert eng.calls[0] == ("edit", "move it", (640, 480)) and eng.calls[1][0] == "ask" and eng.calls[1][2] == 1
    assert (tmp_path / "step" / "images" / "mental_tracking" / "u0_edited.png").exists()
    s = rb.main(["score", "realunify", "--run_dir", str(tmp_path / "step")])
    assert s["samples"] == 2 and s["overall_acc"] == 0.5                          # the engine always answers B
    # interleave mode on two shards, merged by the scorer
    for k in range(2):
        rb.main(["infer", "realunify", "--data_path", str(data), "--output_dir", str(tmp_path / "il"), "--inference_mode",
                 "interleave", "--num_shards", "2", "--shard_rank", str(k), "--target_image_size", "512x512"], engine=eng)
    assert eng.calls[-1][:3] == ("interleave", "Which one? A, B, C or D.", (512, 512))
    assert (tmp_path / "il" / "shards" / "realunify_results_shard_001.jsonl").exists()
    s = rb.main(["score", "realunify", "--run_dir", str(tmp_path / "il")])
    assert s["samples"] == 2 and s["overall_acc"] == 0.5 and s["by_task"]["mental_tracking"]["total"] == 2
    rec = json.loads((tmp_path / "il" / "realunify_results.jsonl").read_text().splitlines()[0])
    assert rec["model_response"] == "C" and len(rec["generated_images"]) == 1 and rec["conversations"][0]["from"] == "system"

    ueg = tmp_path / "ueg.json"
    ueg.write_text(json.dumps([
        {"index": 1, "task_type": "world_knowledge", "new_prompt": "Think first. Here is the prompt for image generation: a red barn\n\nnotes",
         "question_list": [{"question": "Is it red?", "answer": "yes"}, {"question": "Is it a red car?", "answer": "no"}]},
        {"index": 2, "task_type": "code_to_image", "new_prompt": "Here is the prompt for image generation: a plot",
         "question_list": [{"question": "Is it blue?", "answer": "yes"}, {"question": "never asked", "answer": "yes"}]}]))
    eng = _FakeEngine()
    rb.main(["infer", "realunify_ueg", "--data_path", str(ueg), "--output_dir", str(tmp_path / "ueg_t2i"), "--inference_mode", "t2i"], engine=eng)
    assert eng.calls[0] == ("t2i", "a red barn", (1024, 1024))
    rb.main(["infer", "realunify_ueg", "--data_path", str(ueg), "--output_dir", str(tmp_path / "ueg_u"), "--inference_mode",
             "understand_t2i", "--limit", "1"], engine=eng)
    assert eng.calls[-2][0] == "ask" and eng.calls[-1] == ("t2i", "a refined prompt", (1024, 1024))
    judge = _FakeTextJudge()
    s = rb.main(["score", "realunify_ueg", "--run_dir", str(tmp_path / "ueg_t2i")], client=judge)
    assert judge.calls == 3                                                        # the second sample stops at its first miss
    assert s["total"] == {"correct": 0, "total": 2, "accuracy": 0.0}              # "red car" is answered yes as well
    assert s["per_task"]["code_to_image"]["total"] == 1


def test_unimmmu_babyvision_opening_pipelines(tmp_path):
    from evaluation.interleave import run_benchmark as rb
    from evaluation.interleave.suites import BabyVision, rule_answer, split_steps, tagged_answer
    _png(tmp_path / "a.png", (512, 512))
    _png(tmp_path / "b.png", (512, 512))
    uni = tmp_path / "uni.jsonl"
    uni.write_text(json.dumps({"hash_uid": "h1", "id": "maze_3", "task": "maze", "gt_text": "B", "messages": [
        {"role": "user", "content": [{"type": "text", "text": "Solve the maze."}, {"type": "image_url", "image_url": {"url": "a.png"}},
                                     {"type": "image_url", "image_url": {"url": "b.png"}}, {"type": "image_url", "image_url": {"url": "gone.png"}}]}]}) + "\n")
    eng = _FakeEngine()
    rb.main(["infer", "unimmmu", "--data_path", str(uni), "--output_dir", str(tmp_path / "uni"), "--inference_mode", "i2t"], engine=eng)
    assert eng.calls[0] == ("ask", "<image>\n<image>\nSolve the maze.", 2)
    rec = json.loads((tmp_path / "uni" / "unimmmu_results.jsonl").read_text().splitlines()[0])
    assert rec["id"] == "h1" and rec["sample_id"] == "maze_3" and rec["model_response"].startswith("B")
    s = rb.main(["score", "unimmmu", "--run_dir", str(tmp_path / "uni")])
    assert s["samples"] == 1

    assert tagged_answer("<think>x</think>\nso\nB") == "B" and tagged_answer("<answer> 12 </answer> junk") == "12"
    assert rule_answer("thus the answer is: 42") == "42" and rule_answer("no idea") is None
    assert BabyVision.question_and_key({"ansType": "choice", "question": "Q", "options": ["x", "y"], "choiceAns": "2"})[1] == "B"
    assert split_steps("first <image_1> second [image] third") == ["first", "second", "third"]
    bv = tmp_path / "meta_data.jsonl"
    bv.write_text("\n".join(json.dumps(r) for r in [
        {"taskId": 1, "image": "a.png", "question": "How many?", "ansType": "blank", "blankAns": "7", "type": "count", "subtype": "dots"},
        {"taskId": 2, "image": "b.png", "question": "Which?", "ansType": "choice", "options": ["p", "q", "r"], "choiceAns": 3,
         "type": "shape", "subtype": "match"}]))
    rb.main(["infer", "babyvision", "--data_path", str(bv), "--output_dir", str(tmp_path / "bv"), "--workers", "2"], engine=eng)
    judge = _FakeTextJudge()
    s = rb.main(["score", "babyvision", "--run_dir", str(tmp_path / "bv"), "--data_path", str(bv)], client=judge)
    assert judge.calls == 2 and s["samples"] == 2
    scored = [json.loads(l) for l in (tmp_path / "bv" / "babyvision_results_scored.jsonl").read_text().splitlines()]
    assert {r["taskId"]: r["LLMJudgeResult"] for r in scored} == {1: True, 2: False}   # key C, the engine said B

    meta = tmp_path / "opening"
    meta.mkdir()
    _png(meta / "in0.png", (800, 600))
    (meta / "test_data.jsonl").write_text(json.dumps({"total_uid": "T1", "conversations": [
        {"input": [{"text": "<BEGIN> Show how to fold a crane.", "image": "in0.png"}]},
        {"output": [{"text": "fold", "image": "g0.jpg"}, {"text": "crease", "image": "g1.jpg"}]}]}) + "\n")
    rb.main(["infer", "opening", "--meta_path", str(meta), "--output_dir", str(tmp_path / "op"), "--opening_step_prompt_style", "can_be",
             "--max_generation_pixels", str(512 * 512)], engine=eng)
    call = eng.calls[-1]
    assert call[0] == "interleave" and call[1].startswith("The number of generated text-image pairs can be 2: Show how") and call[4] == 2
    assert call[2] == (576, 416)                                                   # 800 x 600 inside 512 x 512 pixels
    saved = json.loads((tmp_path / "op" / "T1.json").read_text())
    assert [o["image"] for o in saved["conversations"][1]["output"]] == ["T1-o-0.jpg", "T1-o-1.jpg"]
    assert [o["text"] for o in saved["conversations"][1]["output"]] == ["step 0", "step 1"] and (tmp_path / "op" / "T1-o-1.jpg").exists()
    s = rb.main(["score", "opening", "--run_dir", str(tmp_path / "op"), "--meta_path", str(meta), "--model_tag", "u1"], client=judge)
    assert s["samples"] == 1 and json.loads((tmp_path / "op" / "opening_summary.json").read_text())["benchmark"] == "opening"


def test_served_engine_speaks_the_servers_dialect():
    import base64, io
    from PIL import Image
    from evaluation.interleave.run_benchmark import ServedEngine, square

    def b64(colour):
        buf = io.BytesIO()
        Image.new("RGB", (8, 8), colour).save(buf, format="PNG")
        return base64.b64encode(buf.getvalue()).decode()

    class Resp:
        def __init__(self, body):
            self.body = body

        def raise_for_status(self):
            pass

        def json(self):
            return self.body

    class Session:
        def __init__(self):
            self.seen = []

        def post(self, url, json=None, timeout=None):
            self.seen.append((url, json))
            if url.endswith("/v1/images/generations") or url.endswith("/v1/images/edits"):
                return Resp({"data": [{"b64_json": b64((1, 2, 3))}]})
            if json.get("interleave"):
                return Resp({"choices": [{"message": {"content": [{"type": "text", "text": "a [image] b"}, {
                    "type": "image_url", "image_url": {"url": "data:image/png;base64," + b64((9, 9, 9))}}]}}]})
            return Resp({"choices": [{"message": {"content": "plain"}}]})

    http = Session()
    eng = ServedEngine("http://h:1/", session=http, cfg_scale=4.0, num_steps=7, seed=3, cfg_interval=(0, 1))
    pic = Image.new("RGB", (8, 8))
    assert eng.t2i("p", (64, 32)).size == (8, 8) and http.seen[-1][1]["size"] == "64x32" and http.seen[-1][1]["num_steps"] == 7
    assert eng.edit("e", [pic], (64, 64)).getpixel((0, 0)) == (1, 2, 3) and len(http.seen[-1][1]["images"]) == 1
    assert eng.ask("q", [pic], max_new_tokens=5) == "plain" and http.seen[-1][1]["max_tokens"] == 5
    big = Image.new("RGB", (100, 60))
    eng.ask("q", [big], min_pixels=64 * 64, max_pixels=64 * 64, repetition_penalty=1.05, do_sample=False, temperature=0)
    sent = http.seen[-1][1]
    got = Image.open(io.BytesIO(base64.b64decode(sent["messages"][0]["content"][1]["image_url"]["url"].split(",", 1)[1])))
    assert got.size[0] % 32 == 0 and got.size[1] % 32 == 0 and got.size[0] * got.size[1] <= 64 * 64
    assert sent["repetition_penalty"] == 1.05 and "temperature" not in sent
    text, pics = eng.interleave("p", [], (64, 64), max_images=2)
    assert text == "a [image] b" and len(pics) == 1 and http.seen[-1][1]["max_rounds"] == 2
    assert square("1024x1024") == 1024 and square("512") == 512
    with pytest.raises(Exception):
        square("640x480")


def test_evalscope_launcher_resolves_its_configuration(monkeypatch):
    import importlib.util
    root = Path(__file__).resolve().parents[1]
    spec = importlib.util.spec_from_file_location("run_evalscope", root / "evaluation" / "understanding" / "run_evalscope.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    monkeypatch.setenv("JUDGE_API_KEY", "k")
    cfg = mod.main(["--dry_run", "--api_url", "http://h:1/v1/", "--datasets", "ai2d", "--no_thinking", "--limit", "5"])
    assert cfg["api_url"] == "http://h:1/v1/" and cfg["datasets"] == ["ai2d"] and cfg["limit"] == 5
    assert cfg["generation_config"]["extra_body"]["chat_template_kwargs"]["enable_thinking"] is False
    assert "remove_until" not in cfg["dataset_args"] and cfg["judge_model_args"]["api_key"] == "k"
    full = mod.main(["--dry_run"])
    assert full["datasets"] == ["mmmu_pro", "mmlu_pro", "mm_bench", "ai2d", "math_vista", "ifeval"]
    assert full["generation_config"]["temperature"] == 0.6 and full["dataset_args"]["remove_until"] == "</think>"
    spec = importlib.util.spec_from_file_location("sensenova_models", root / "evaluation" / "easi" / "sensenova_models.py")
    m2 = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m2)
    assert isinstance(m2.entries, dict)


def test_repeated_runs_are_reported_as_mean_and_std(tmp_path, capsys):
    from evaluation.benchmarks import score
    runs = [[{"LLMJudgeResult": True, "Type": "Visual Tracking", "Subtype": "maze"}, {"LLMJudgeResult": ok, "Type": "Visual Tracking", "Subtype": "maze"}]
            for ok in (True, False)]
    files = []
    for i, recs in enumerate(runs):
        f = tmp_path / f"run{i}.jsonl"
        f.write_text("\n".join(json.dumps(r) for r in recs))
        files.append(str(f))
    assert score.main(["--benchmark", "babyvision", "--records", *files, "--out", str(tmp_path / "s.json")]) == 0
    s = json.loads((tmp_path / "s.json").read_text())
    assert s["runs"] == 2 and s["across_runs"]["overall_accuracy"] == {"mean": 0.75, "std": 0.25}
    assert s["across_runs"]["by_type"]["Visual Tracking"]["accuracy"]["mean"] == 0.75 and len(s["per_run"]) == 2
    assert score.across_runs([{"a": 1, "b": "x"}, {"a": 3, "c": 2}]) == {"a": {"mean": 2.0, "std": 1.0}}


def test_tiif_dimension_table():
    from evaluation.benchmarks.rules import TIIF_DIMENSIONS, tiif_summary
    assert sum(len(v) for d in TIIF_DIMENSIONS.values() for v in d.values()) == 4 + 4 + 4 + 8 + 8 + 8 + 1 + 1 + 1
    recs = [{"attribute": "numeracy", "type": "short", "gt_answers": ["yes", "no"], "model_pred": ["yes", "yes"]},
            {"attribute": "text", "type": "short", "gt_answers": ["yes"], "model_pred": ["yes"]},
            {"attribute": "text", "type": "long", "gt_answers": ["no"], "model_pred": ["yes"]}]
    s = tiif_summary(recs)
    assert s["dimensions"]["Basic/Reasoning"] == {"short": 0.5, "long": None}
    assert s["dimensions"]["Advanced/Overall"] == {"short": 1.0, "long": 0.0}
    assert s["overall"] == {"short": 0.75, "long": 0.0}                 # mean over the dimensions that have pictures
