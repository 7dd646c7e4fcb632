"""Random Sanesun configurations (layer order, head layouts, sizes on and off the tensor-core grid, windows, taps,
latent widths): the ragged step engine in fp32 and bf16, two requests cut into random portions and mixed in steps,
against oracle/sanesun_ref.py.  ``python tools/fuzz_sanesun.py [n_seeds]`` on a B200; prints one line per seed and
``bad <count>``."""
import sys, random, math, json, traceback
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import dgi_b200
from dgi_b200 import sanesun_layer as S
from dgi_b200.ragged_engine import RaggedStepEngine
from oracle import sanesun_ref as R

def rand_cfg(rng):
    W = rng.choice([32, 48, 64, 96, 128])
    layers = []
    for _ in range(rng.randint(2, 6)):
        kind = rng.choice(S.MIXERS)
        if kind == 'attention':
            G = rng.choice([1, 2, 3, 4]); H = G * rng.choice([1, 2, 3, 4])
            dk = rng.choice([8, 16, 24, 32, 48, 64, 128]); dv = rng.choice([8, 16, 24, 32, 48, 64, 96, 128, 2 * rng.randint(2, 40)])
            dims = rng.choice([2, 4, dk // 2 - (dk // 2) % 2, dk])
            m = {'heads': H, 'kv_heads': G, 'dim': dk, 'vdim': dv, 'scale': rng.choice([dk ** -0.5, 0.1, 0.3]),
                 'mask': {'size': rng.choice([1, 2, 7, 16, 31, 32, 33, 64, 100]), 'keep_first': rng.choice([0, 1, 3, 16, 20, 40])},
                 'rot': {'base': rng.choice([50.0, 10000.0, 1e6]), 'dims': max(2, dims)}}
        elif kind == 'latent_attention':
            H = rng.choice([1, 2, 3, 5, 8, 12]); dk = rng.choice([4, 8, 16, 32, 64]); dv = rng.choice([4, 8, 24, 48, 64])
            m = {'heads': H, 'dim': dk, 'vdim': dv, 'kv_rank': rng.choice([8, 16, 24, 32, 48, 64, 80, 128, 256, 272]),
                 'q_rank': rng.choice([8, 24, 96]), 'scale': rng.choice([dk ** -0.5, 0.2])}
        else:
            G = rng.choice([1, 2, 3]); H = G * rng.choice([1, 2, 3])
            m = {'heads': H, 'kv_heads': G, 'dim': rng.choice([4, 8, 16, 32, 33, 64, 96, 128, 160]), 'vdim': rng.choice([4, 16, 31, 32, 64, 100]),
                 'conv': rng.choice([1, 2, 3, 4, 5, 8])}
        layers.append({'type': kind, 'mixer': m, 'mlp': rng.choice([None, {'kind': 'dense', 'ff': rng.choice([8, 40, 136, 320])}])})
    return {'architecture': 'Sanesun', 'width': W, 'vocab': rng.choice([17, 64, 301]), 'embedding': {'scale': rng.choice([1.0, 4.0, 16.0])},
            'norm': {'eps': rng.choice([1e-6, 1e-5])}, 'layers': layers}

bad = 0
for seed in range(int(sys.argv[1]) if len(sys.argv) > 1 else 24):
    rng = random.Random(seed)
    raw = rand_cfg(rng)
    try:
        cfg = S.SanesunConfig.from_dict(raw)
        tensors = S.random_checkpoint(cfg, seed=seed)
        g = torch.Generator().manual_seed(seed)
        n1, n2 = rng.randint(40, 150), rng.randint(1, 60)
        t1 = torch.randint(0, raw['vocab'], (n1,), generator=g).tolist(); t2 = torch.randint(0, raw['vocab'], (n2,), generator=g).tolist()
        ref1, ref2 = R.forward(raw, tensors, t1), R.forward(raw, tensors, t2)
        for dt, tol in ((torch.float32, 5e-5), (torch.bfloat16, 6e-2)):
            eng = RaggedStepEngine(S.build_shards(cfg, tensors, [(0, cfg.num_hidden_layers)], 'cuda:0', dt), max_tokens=256, max_seqs=2)
            got1, got2, a1, a2 = [], [], 0, 0
            while a1 < n1 or a2 < n2:
                entries = []
                c1 = min(n1 - a1, rng.choice([1, 1, 2, 3, 17, 40])); c2 = min(n2 - a2, rng.choice([0, 1, 2, 9]))
                if c1: entries.append(('a', t1[a1:a1 + c1], list(range(c1))))
                if c2: entries.append(('b', t2[a2:a2 + c2], list(range(c2))))
                if rng.random() < 0.5: entries.reverse()
                out = eng.step(entries); o = 0
                for rid, toks, _ in entries:
                    (got1 if rid == 'a' else got2).append(out[o:o + len(toks)]); o += len(toks)
                a1 += c1; a2 += c2
            eng.release()
            for got, ref in ((got1, ref1), (got2, ref2)):
                gg = torch.cat(got).cpu().double()
                if dt == torch.float32:
                    err = float((gg - ref).abs().max() / max(1.0, ref.abs().max()))
                else:
                    err = float((gg - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())
                if not (err <= tol):
                    bad += 1
                    print('MISMATCH seed', seed, dt, err, json.dumps(raw), flush=True)
        print('seed', seed, 'ok', [(l['type'][:3], l['mixer'].get('dim'), l['mixer'].get('vdim')) for l in raw['layers']], flush=True)
    except Exception as e:
        bad += 1
        print('ERROR seed', seed, type(e).__name__, str(e)[:300], json.dumps(raw), flush=True)
        traceback.print_exc()
print('bad', bad)
