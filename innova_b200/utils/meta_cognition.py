"""``MetaCognitionEngine``: reasoning-chain analysis, confidence calibration, goal decomposition, strategy selection and the
feedback loop that turns a record of past tasks into a self assessment (reference: include/oil/meta_cognition.h:14-156,
src/meta_cognition.cpp:55-725).

The decision rules (thresholds for an inconsistent step, the keyword table that picks a strategy, the weights of the overall
score) are the reference's. The model-backed parts run on a torch model callable as ``model(ids) -> logits [B, S, V]`` with a
``cfg.vocab_size``: the per-step entropy is taken from ONE batched forward over the output's bytes on the model's device
(softmax and entropy in fp32), and text is generated greedily with the same byte codec as the rest of the ASI classes.
Without a model every method still answers, with the reference's fixed fallbacks.
"""
from __future__ import annotations

import enum
import math
import time
from collections import Counter
from dataclasses import dataclass, field
from typing import Dict, List

import torch

from .asi_ext import simple_decode, simple_encode


class ReasoningStrategy(enum.IntEnum):
    FORWARD = 0
    BACKWARD = 1
    ANALOGICAL = 2
    DECOMPOSITION = 3
    HYPOTHETICAL = 4


@dataclass
class ReasoningStep:
    description: str = ""
    confidence: float = 0.0
    entropy: float = 0.0
    consistent: bool = True
    step_index: int = 0
    strategy_used: ReasoningStrategy = ReasoningStrategy.FORWARD


@dataclass
class ReasoningChain:
    steps: List[ReasoningStep] = field(default_factory=list)
    overall_confidence: float = 0.0
    consistency_score: float = 0.0
    inconsistency_count: int = 0
    chain_id: int = 0
    goal: str = ""


@dataclass
class ConfidenceRecord:
    predicted_confidence: float = 0.0
    was_correct: bool = False
    task_description: str = ""
    timestamp: int = 0


@dataclass
class CalibrationBin:
    bin_lower: float = 0.0
    bin_upper: float = 0.0
    total_count: int = 0
    correct_count: int = 0
    avg_confidence: float = 0.0


@dataclass
class SubGoal:
    description: str = ""
    estimated_difficulty: float = 0.0
    depends_on: List[int] = field(default_factory=list)
    completed: bool = False
    failed: bool = False
    result: str = ""
    subgoal_id: int = 0


@dataclass
class GoalDecomposition:
    original_goal: str = ""
    subgoals: List[SubGoal] = field(default_factory=list)
    total_subgoals: int = 0
    completed_subgoals: int = 0
    progress: float = 0.0


@dataclass
class MetacognitiveInsight:
    insight_text: str = ""
    relevance_score: float = 0.0
    timestamp: int = 0
    source_task: str = ""


@dataclass
class SelfAssessment:
    accuracy_score: float = 0.0
    speed_score: float = 0.0
    resource_efficiency: float = 0.0
    overall_score: float = 0.0
    tasks_evaluated: int = 0
    avg_confidence: float = 0.0
    avg_calibration_error: float = 0.0


@dataclass
class FeedbackEntry:
    task: str = ""
    strategy_used: str = ""
    performance_score: float = 0.0
    succeeded: bool = False
    failure_reason: str = ""
    duration_ms: int = 0


_DEPENDENCY_MARKERS = ("depends on:", "requires:", "after:")

# (keywords, strategy) in the order they are tried; difficulty > 0.7 also selects DECOMPOSITION at the third rule
_STRATEGY_RULES = (
    (("why", "cause", "reason"), ReasoningStrategy.BACKWARD),
    (("similar", "like", "analogy"), ReasoningStrategy.ANALOGICAL),
    (("decompose", "break down", "steps"), ReasoningStrategy.DECOMPOSITION),
    (("what if", "suppose", "imagine"), ReasoningStrategy.HYPOTHETICAL),
)

_TASK_TYPES = (
    ("code", ("code", "program", "function")),
    ("math", ("math", "calculate", "equation")),
    ("explanation", ("explain", "why")),
    ("planning", ("plan", "strategy")),
    ("creative", ("write", "story")),
)

_STRATEGY_AFFINITY = {
    ReasoningStrategy.FORWARD: (("compute", "calculate"), 0.5),
    ReasoningStrategy.BACKWARD: (("why", "explain"), 0.4),
    ReasoningStrategy.ANALOGICAL: (("compare", "similar"), 0.3),
    ReasoningStrategy.DECOMPOSITION: (("complex", "plan"), 0.5),
    ReasoningStrategy.HYPOTHETICAL: (("what if", "imagine"), 0.3),
}


def _trim(history: list, limit: int):
    if len(history) > limit:
        del history[: len(history) - limit]


class MetaCognitionEngine:
    max_history = 10000
    max_confidence_records = 50000

    def __init__(self, model=None):
        self.model = model
        self._chains: List[ReasoningChain] = []
        self._confidence: List[ConfidenceRecord] = []
        self._feedback: List[FeedbackEntry] = []
        self._insights: List[MetacognitiveInsight] = []
        self._next_chain_id = 0
        self._next_subgoal_id = 0

    # ------------------------------------------------------------------------------------------ model access
    def _vocab(self) -> int:
        return int(self.model.cfg.vocab_size)

    def _device(self):
        try:
            return next(self.model.parameters()).device
        except (StopIteration, AttributeError):
            return torch.device("cpu")

    @torch.no_grad()
    def _generate(self, prompt: str, max_new: int) -> str:
        """Greedy continuation of ``prompt``; the context is cut to the model's window from the left."""
        vocab = self._vocab()
        ids = simple_encode(prompt, vocab)
        window = int(getattr(self.model.cfg, "max_seq_len", getattr(self.model.cfg, "seq_len", 1024)))
        dev = self._device()
        out: List[int] = []
        for _ in range(max(0, max_new)):
            ctx = (ids + out)[-window:]
            logits = self.model(torch.tensor([ctx], device=dev))[0, -1].float()
            out.append(int(torch.argmax(logits)))
        return simple_decode(out)

    @torch.no_grad()
    def _position_entropies(self, text: str) -> List[float]:
        """Normalised entropy (0 = certain, 1 = uniform) of the model's next-token distribution at each of the first 64
        bytes of ``text``."""
        vocab = self._vocab()
        n = min(64, max(1, len(text)))
        raw = text.encode("utf-8", "replace") or b" "
        ids = [min(raw[i % len(raw)], vocab - 1) for i in range(n)]
        logits = self.model(torch.tensor([ids], device=self._device()))[0].float()
        logp = torch.log_softmax(logits, dim=-1)
        ent = -(logp.exp() * logp).sum(-1)
        norm = math.log(logits.shape[-1]) if logits.shape[-1] > 1 else 1.0
        return (ent / norm).clamp(0.0, 1.0).tolist()

    # ------------------------------------------------------------------------------------------ reasoning chains
    def analyze_reasoning(self, input: str, output: str) -> ReasoningChain:   # noqa: A002 - the reference's argument name
        chain = ReasoningChain(chain_id=self._next_chain_id, goal=input)
        self._next_chain_id += 1
        if self.model is None:
            chain.steps.append(ReasoningStep(description=output or "no model available", confidence=0.0, entropy=1.0))
            chain.consistency_score = 1.0
            self._chains.append(chain)
            return chain

        analysis = self._generate(
            f"Analyze the reasoning in this output for the goal: {input}\nOutput: {output}\n"
            "Break down into steps and rate each step's confidence (0-1):", 100)
        entropies = self._position_entropies(output)
        for line in analysis.split("\n"):
            if len(chain.steps) >= 50:
                break
            if not line:
                continue
            idx = len(chain.steps)
            ent = entropies[idx % len(entropies)]
            step = ReasoningStep(description=line, confidence=1.0 - ent, entropy=ent, step_index=idx,
                                 strategy_used=self.select_strategy(line, 0.5))
            if chain.steps:
                step.consistent = self.check_step_consistency(chain.steps[-1], step)
                chain.inconsistency_count += not step.consistent
            chain.steps.append(step)
        if chain.steps:
            chain.overall_confidence = sum(s.confidence for s in chain.steps) / len(chain.steps)
        else:
            chain.steps.append(ReasoningStep(description="analysis: " + output, confidence=0.5, entropy=0.5))
            chain.overall_confidence = 0.5
        chain.consistency_score = self.calculate_chain_consistency(chain)
        self._chains.append(chain)
        _trim(self._chains, self.max_history)
        return chain

    @staticmethod
    def check_step_consistency(prev: ReasoningStep, curr: ReasoningStep) -> bool:
        """A step breaks the chain when confidence falls by more than 0.4 or a focused step is followed by a diffuse one."""
        if prev.confidence - curr.confidence > 0.4:
            return False
        return not (curr.entropy > 0.8 and prev.entropy < 0.3)

    @staticmethod
    def calculate_chain_consistency(chain: ReasoningChain) -> float:
        pairs = len(chain.steps) - 1
        if pairs <= 0:
            return 1.0
        return sum(1 for s in chain.steps[1:] if s.consistent) / pairs

    def identify_reasoning_errors(self, chain: ReasoningChain) -> None:
        """Marks steps inconsistent on three separate grounds (very low confidence, entropy jump, confidence drop > 0.5);
        each ground that applies adds one to ``inconsistency_count``."""
        for prev, curr in zip(chain.steps, chain.steps[1:]):
            grounds = (curr.confidence < 0.2) + (curr.entropy > 0.7 and prev.entropy < 0.3) \
                + (prev.confidence - curr.confidence > 0.5)
            if grounds:
                curr.consistent = False
                chain.inconsistency_count += grounds
        chain.consistency_score = self.calculate_chain_consistency(chain)

    @staticmethod
    def find_first_error_step(chain: ReasoningChain) -> int:
        return next((s.step_index for s in chain.steps if not s.consistent), -1)

    @staticmethod
    def diagnose_error(chain: ReasoningChain, error_step: int) -> str:
        if not 0 <= error_step < len(chain.steps):
            return f"No error at step {error_step}"
        step = chain.steps[error_step]
        lines = [f"Error at step {error_step}:", f"  Description: {step.description}",
                 f"  Confidence: {step.confidence:g}", f"  Entropy: {step.entropy:g}"]
        if step.confidence < 0.3:
            lines.append("  Diagnosis: LOW CONFIDENCE - model is uncertain about this step")
        if step.entropy > 0.7:
            lines.append("  Diagnosis: HIGH ENTROPY - reasoning is diffuse, not focused")
        if error_step > 0:
            drop = chain.steps[error_step - 1].confidence - step.confidence
            if drop > 0.4:
                lines.append(f"  Diagnosis: SHARP CONFIDENCE DROP from step {error_step - 1} ({drop:g} drop)")
        return "\n".join(lines) + "\n"

    # ------------------------------------------------------------------------------------------ calibration
    def record_confidence(self, predicted: float, correct: bool, task: str = "") -> None:
        self._confidence.append(ConfidenceRecord(float(predicted), bool(correct), task, int(time.time())))
        _trim(self._confidence, self.max_confidence_records)

    def get_calibration_bins(self, num_bins: int = 10) -> List[CalibrationBin]:
        width = 1.0 / num_bins
        bins = [CalibrationBin(i * width, (i + 1) * width) for i in range(num_bins)]
        for rec in self._confidence:
            b = bins[min(num_bins - 1, max(0, int(rec.predicted_confidence / width)))]
            b.total_count += 1
            b.correct_count += rec.was_correct
            b.avg_confidence += rec.predicted_confidence
        for b in bins:
            if b.total_count:
                b.avg_confidence /= b.total_count
        return bins

    def get_expected_calibration_error(self) -> float:
        bins = [b for b in self.get_calibration_bins(10) if b.total_count]
        total = sum(b.total_count for b in bins)
        if not total:
            return 0.0
        return sum(abs(b.avg_confidence - b.correct_count / b.total_count) * b.total_count for b in bins) / total

    def get_current_confidence(self) -> float:
        recent = self._confidence[-100:]
        if not recent:
            return 0.5
        return sum(r.predicted_confidence for r in recent) / len(recent)

    # ------------------------------------------------------------------------------------------ goals
    def _new_subgoal(self, **kw) -> SubGoal:
        sg = SubGoal(subgoal_id=self._next_subgoal_id, **kw)
        self._next_subgoal_id += 1
        return sg

    def decompose_goal(self, goal: str, max_subgoals: int = 20) -> GoalDecomposition:
        decomp = GoalDecomposition(original_goal=goal)
        if self.model is None:
            for verb, difficulty in (("Analyze", 0.3), ("Execute", 0.6), ("Verify", 0.4)):
                deps = [decomp.subgoals[-1].subgoal_id] if decomp.subgoals else []
                decomp.subgoals.append(self._new_subgoal(description=f"{verb}: {goal}", estimated_difficulty=difficulty,
                                                         depends_on=deps))
            decomp.total_subgoals = 3
            return decomp

        text = self._generate(f"Decompose this goal into subgoals with dependencies:\n{goal}\n"
                              "List each subgoal with its prerequisites (if any):", max_subgoals * 10)
        by_line: Dict[str, int] = {}
        for line in text.split("\n"):
            if len(decomp.subgoals) >= max_subgoals:
                break
            if not line:
                continue
            sg = self._new_subgoal(description=line)
            marker = next((m for m in _DEPENDENCY_MARKERS if m in line), None)
            if marker is not None:
                at = line.index(marker)
                sg.description = line[:at]
                # an earlier subgoal is a prerequisite when its line occurs inside one of the words after the marker
                for word in line[at + len(marker):].split():
                    sg.depends_on.extend(i for name, i in by_line.items() if name in word)
            sg.estimated_difficulty = 0.3 + (len(sg.description) % 50) / 100.0
            by_line[line] = sg.subgoal_id
            decomp.subgoals.append(sg)
        if not decomp.subgoals:
            decomp.subgoals.append(self._new_subgoal(description=goal, estimated_difficulty=0.5))
        decomp.total_subgoals = len(decomp.subgoals)
        return decomp

    @staticmethod
    def check_subgoal_completion(decomp: GoalDecomposition) -> bool:
        return all(sg.completed or sg.failed for sg in decomp.subgoals)

    @staticmethod
    def get_ready_subgoals(decomp: GoalDecomposition) -> List[int]:
        done = {sg.subgoal_id for sg in decomp.subgoals if sg.completed}
        return [sg.subgoal_id for sg in decomp.subgoals
                if not (sg.completed or sg.failed) and all(d in done for d in sg.depends_on)]

    # ------------------------------------------------------------------------------------------ strategies
    @staticmethod
    def select_strategy(task: str, difficulty: float) -> ReasoningStrategy:
        low = task.lower()
        for keywords, strategy in _STRATEGY_RULES:
            if any(k in low for k in keywords):
                return strategy
            if strategy is ReasoningStrategy.DECOMPOSITION and difficulty > 0.7:
                return strategy
        return ReasoningStrategy.DECOMPOSITION if difficulty > 0.6 else ReasoningStrategy.FORWARD

    def get_best_strategy_for_task_type(self, task_type: str) -> ReasoningStrategy:
        """The strategy with the most recorded successes; each successful entry's ``strategy_used`` text is mapped to a
        strategy through the keyword table. ``task_type`` does not filter the history (nor does it in the reference)."""
        wins = Counter(self.select_strategy(fb.strategy_used, 0.5) for fb in self._feedback if fb.succeeded)
        if not wins:
            return ReasoningStrategy.FORWARD
        top = max(wins.values())
        return min(s for s, c in wins.items() if c == top)

    @staticmethod
    def extract_task_type_score(task: str, strategy: ReasoningStrategy) -> float:
        keywords, base = _STRATEGY_AFFINITY[strategy]
        return 0.8 if any(k in task.lower() for k in keywords) else base

    @staticmethod
    def task_type_classify(task: str) -> str:
        low = task.lower()
        return next((name for name, keys in _TASK_TYPES if any(k in low for k in keys)), "general")

    # ------------------------------------------------------------------------------------------ feedback loop
    def record_feedback(self, entry: FeedbackEntry) -> None:
        self._feedback.append(entry)
        _trim(self._feedback, self.max_history)

    def get_recent_feedback(self, count: int = 50) -> List[FeedbackEntry]:
        return list(self._feedback[-count:]) if count > 0 else []

    def generate_feedback_summary(self) -> str:
        if not self._feedback:
            return "No feedback recorded yet."
        total = len(self._feedback)
        wins = sum(fb.succeeded for fb in self._feedback)
        used = Counter(fb.strategy_used for fb in self._feedback)
        won = Counter(fb.strategy_used for fb in self._feedback if fb.succeeded)
        lines = ["Metacognitive Feedback Summary", f"  Total tasks: {total}",
                 f"  Successes: {wins} ({wins / total * 100:g}%)",
                 f"  Average performance: {sum(fb.performance_score for fb in self._feedback) / total:g}",
                 "", "Strategy breakdown:"]
        lines += [f"  {s}: {won[s]}/{n} ({won[s] / n * 100:g}%)" for s, n in used.items()]
        return "\n".join(lines) + "\n"

    def extract_improvement_patterns(self) -> List[str]:
        if len(self._feedback) < 10:
            return []
        recent = self._feedback[-50:]
        fails = Counter(fb.strategy_used for fb in recent if not fb.succeeded)
        wins = Counter(fb.strategy_used for fb in recent if fb.succeeded)
        patterns = [f"Strategy '{s}' has high failure rate ({f} fails vs {wins[s]} wins) - consider alternative"
                    for s, f in fails.items() if f > 2 * wins[s]]
        reasons = Counter(fb.failure_reason for fb in recent if not fb.succeeded and fb.failure_reason)
        patterns += [f"Recurring failure: '{r}' (occurred {c} times)" for r, c in reasons.items() if c >= 3]
        return patterns

    def assess_self(self, lookback_count: int = 100) -> SelfAssessment:
        window = self._feedback[-lookback_count:] if lookback_count > 0 else []
        a = SelfAssessment()
        if not window:
            return a
        n = len(window)
        a.tasks_evaluated = n
        a.accuracy_score = sum(fb.succeeded for fb in window) / n
        a.speed_score = 1.0 / (1.0 + sum(fb.duration_ms for fb in window) / n / 1000.0)
        a.resource_efficiency = 1.0 - len(self._feedback) / self.max_history
        a.avg_confidence = self.get_current_confidence()
        a.avg_calibration_error = self.get_expected_calibration_error()
        a.overall_score = (0.4 * a.accuracy_score + 0.2 * a.speed_score + 0.15 * a.resource_efficiency
                           + 0.25 * (1.0 - a.avg_calibration_error))
        return a

    def generate_insight(self, task: str, result: str = "") -> MetacognitiveInsight:
        a = self.assess_self(50)
        if a.avg_calibration_error > 0.2:
            lean = "overconfident" if a.avg_confidence > a.accuracy_score else "underconfident"
            text, score = f"Confidence calibration is off by {a.avg_calibration_error:.6f} — tend to {lean}", \
                a.avg_calibration_error
        elif a.accuracy_score < 0.5:
            text, score = f"Accuracy is low ({a.accuracy_score:.6f}) — consider more deliberate reasoning strategies", \
                1.0 - a.accuracy_score
        elif a.accuracy_score > 0.8:
            text, score = f"Performance is strong ({a.accuracy_score:.6f}) — can take on more complex tasks", \
                0.5 * a.accuracy_score
        else:
            text, score = f"Task type '{self.task_type_classify(task)}' — current overall score: {a.overall_score:.6f}", 0.5
        insight = MetacognitiveInsight(text, score, int(time.time()), task)
        self._insights.append(insight)
        _trim(self._insights, self.max_history)
        return insight

    # ------------------------------------------------------------------------------------------ accessors
    def get_history(self) -> List[ReasoningChain]:
        return list(self._chains)

    def get_confidence_history(self) -> List[ConfidenceRecord]:
        return list(self._confidence)

    def get_insights(self) -> List[MetacognitiveInsight]:
        return list(self._insights)

    def reset(self) -> None:
        self._chains.clear()
        self._confidence.clear()
        self._feedback.clear()
        self._insights.clear()
        self._next_chain_id = 0
        self._next_subgoal_id = 0
