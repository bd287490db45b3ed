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
