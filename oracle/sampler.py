"""TEST INFRASTRUCTURE ONLY — a CPU restatement of the reference's token sampler, the checker of the library's
`spl_topk` / `spl_sample_topk` / `spl_sampler_distribution` / `spl_speculative_resolve`. Nothing shipped imports it.

Follows Sources/SploshRuntime/Sampler.swift: TopK.select (:19-52), Sampler.uniform (:79-90), distribution (:100-116),
draw (:119-126), sample (:128-156), SpeculativeSampling.resolve (:163-179). Arithmetic is single precision, in the
reference's order of operations (numpy float32 scalars).

Parity unpinned: the reference holds no test or stored vector for its sampler (Tests/ has none that mentions it),
so this restatement is checked only against the source it follows."""
import numpy as np

F = np.float32
MASK = (1 << 64) - 1


def topk_select(logits, limit, k):
    """The k largest of logits[:limit] in descending order, lower index first among equals; slots that nothing
    fills stay (0, -inf)."""
    ids = [0] * k
    values = [F(-np.inf)] * k
    for index in range(limit):
        value = F(logits[index])
        if not value > values[k - 1]:
            continue
        slot = k - 1
        while slot > 0 and values[slot - 1] < value:
            values[slot] = values[slot - 1]; ids[slot] = ids[slot - 1]; slot -= 1
        values[slot] = value; ids[slot] = index
    return ids, np.array(values, F)


class Sampler:
    def __init__(self, temperature=1.0, top_p=0.95, top_k=20, seed=1):
        self.temperature, self.top_p, self.top_k, self.state = F(temperature), F(top_p), int(top_k), int(seed) & MASK

    def uniform(self):
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        z ^= z >> 31
        return F(z >> 40) / F(1 << 24)

    def _softmax(self, values, temperature):
        top = F(values[0])
        probabilities = [F(np.exp((F(v) - top) / temperature)) for v in values]
        total = F(0)
        for p in probabilities:
            total = F(total + p)
        return [F(p / total) for p in probabilities]

    def _kept(self, probabilities):
        kept = len(probabilities)
        if self.top_p < 1:
            mass = F(0)
            for index, p in enumerate(probabilities):
                mass = F(mass + p)
                if mass >= self.top_p:
                    kept = index + 1
                    break
        return kept

    def sample(self, ids, values):
        if self.temperature <= 0:
            return int(ids[0])
        probabilities = self._softmax(values, self.temperature)
        kept = self._kept(probabilities)
        kept_mass = F(0)
        for p in probabilities[:kept]:
            kept_mass = F(kept_mass + p)
        draw = F(self.uniform() * kept_mass)
        for index in range(kept):
            draw = F(draw - probabilities[index])
            if draw <= 0:
                return int(ids[index])
        return int(ids[kept - 1])

    def distribution(self, ids, values):
        probabilities = self._softmax(values, max(self.temperature, F(1e-6)))
        kept = self._kept(probabilities)
        total = F(0)
        for p in probabilities[:kept]:
            total = F(total + p)
        return list(ids[:kept]), np.array([F(p / total) for p in probabilities[:kept]], F)

    def draw(self, probabilities):
        remaining = self.uniform()
        for index, p in enumerate(probabilities):
            remaining = F(remaining - F(p))
            if remaining <= 0:
                return index
        return len(probabilities) - 1

    def resolve(self, draft, candidates, draft_probabilities, target_ids, target_probabilities):
        candidates, target_ids = list(candidates), list(target_ids)
        q = F(draft_probabilities[candidates.index(draft)]) if draft in candidates else F(0)
        p = F(target_probabilities[target_ids.index(draft)]) if draft in target_ids else F(0)
        if F(self.uniform() * q) < p:
            return None
        residual = [F(x) for x in target_probabilities]
        for slot, token in enumerate(target_ids):
            if token in candidates:
                residual[slot] = max(F(0), F(residual[slot] - F(draft_probabilities[candidates.index(token)])))
        total = F(0)
        for r in residual:
            total = F(total + r)
        residual = [F(r / total) for r in residual] if total > 0 else [F(x) for x in target_probabilities]
        return int(target_ids[self.draw(residual)])
