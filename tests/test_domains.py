"""Vision / text / audio / RL packages on CPU (reference: vision/*_test.go, text/*_test.go,
audio/*_test.go, rl/*_test.go)."""
import math
import os

import torch

import mimir_b200.tensor as T
from mimir_b200 import audio, nn, rl, text, vision


def test_resnet_mobilenet_vit_unet_shapes_and_gradients():
    nn.manual_seed(0)
    x = T.from_torch(torch.randn(2, 3, 64, 64))
    for make, params in ((lambda: vision.resnet18(10), 11.18e6), (lambda: vision.resnet50(10), 23.5e6),
                         (lambda: vision.MobileNetV2(10), 2.2e6)):
        m = make()
        n = sum(p.value().numel() for p in m.parameters())
        assert abs(n - params) / params < 0.05, n
        assert tuple(m(x).shape) == (2, 10)
    assert len(vision.resnet34().blocks) == 16
    v = vision.ViT(image=32, patch=8, dim=32, depth=2, heads=2, mlp=64, classes=5)
    y = v(T.from_torch(torch.randn(2, 3, 32, 32)))
    assert tuple(y.shape) == (2, 5)
    T.backward(T.mean(y * y))
    assert v.cls.grad() is not None and float(v.patch.weight.grad().data().abs().sum()) > 0
    u = vision.UNet(3, 2, width=4, depth=2)
    assert tuple(u(T.from_torch(torch.randn(1, 3, 16, 16))).shape) == (1, 2, 16, 16)


def test_centernet_heads_loss_decode():
    nn.manual_seed(0)
    net = vision.CenterNet(classes=3, backbone=vision.resnet18(width=8))
    heat, size, off = net(T.from_torch(torch.randn(1, 3, 64, 64)))
    assert tuple(heat.shape) == (1, 3, 16, 16) and tuple(size.shape) == (1, 2, 16, 16)
    th = torch.zeros(1, 3, 16, 16); th[0, 1, 4, 5] = 1
    mask = torch.zeros(1, 16, 16); mask[0, 4, 5] = 1
    loss = vision.centernet_loss(heat, size, off, T.from_torch(th), T.from_torch(torch.zeros(1, 2, 16, 16)),
                                 T.from_torch(torch.zeros(1, 2, 16, 16)), T.from_torch(mask))
    assert math.isfinite(float(loss.data()))
    h = torch.full((1, 3, 16, 16), -10.0); h[0, 2, 7, 3] = 10
    boxes, scores, cls = vision.centernet_decode(h, torch.full((1, 2, 16, 16), 2.0), torch.zeros(1, 2, 16, 16), k=5)
    assert cls[0, 0] == 2 and torch.allclose(boxes[0, 0], torch.tensor([8.0, 24, 16, 32]))


def test_boxes():
    a = torch.tensor([[0.0, 0, 10, 10], [1, 1, 11, 11], [50, 50, 60, 60]])
    iou = vision.box_iou(a, a)
    assert torch.allclose(iou.diag(), torch.ones(3)) and abs(iou[0, 1] - 81 / 119) < 1e-5
    assert vision.nms(a, torch.tensor([0.9, 0.8, 0.7]), 0.5).tolist() == [0, 2]
    assert abs(vision.average_precision(a, torch.tensor([0.9, 0.8, 0.7]), a[[0, 2]]) - (0.5 + 0.5 * 2 / 3)) < 1e-6


def test_wordpiece_and_bert():
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "the", "un", "##aff", "##able", "cat", ",", "##s", "run", "##ning"]
    wp = text.WordPiece(vocab)
    assert wp.tokenize("The unaffable cats, running!") == ["the", "un", "##aff", "##able", "cat", "##s", ",", "run", "##ning", "[UNK]"]
    ids, types, mask = wp.encode("the cat", "cats", max_len=10)
    assert ids[:7] == [2, 5, 9, 3, 9, 11, 3] and types[:7] == [0, 0, 0, 0, 1, 1, 1] and mask == [1] * 7 + [0] * 3
    assert wp.decode(ids) == "the cat cats"
    nn.manual_seed(0)
    cfg = text.BertConfig.tiny(len(vocab))
    m = text.BertForMaskedLM(cfg).eval()
    tid = T.from_torch(torch.tensor([ids]))
    logits = m(tid, T.from_torch(torch.tensor([types])), T.from_torch(torch.tensor([mask])))
    assert tuple(logits.shape) == (1, 10, len(vocab))
    # padding positions do not influence the real ones
    ids2 = list(ids); ids2[-1] = 7
    logits2 = m(T.from_torch(torch.tensor([ids2])), T.from_torch(torch.tensor([types])), T.from_torch(torch.tensor([mask])))
    assert torch.allclose(logits.data()[0, :7], logits2.data()[0, :7], atol=1e-5)
    c = text.BertForSequenceClassification(cfg, 3).eval()
    assert tuple(c(tid).shape) == (1, 3)


def test_audio_front_end(tmp_path):
    rate = 16000
    t = torch.arange(rate) / rate
    x = 0.5 * torch.sin(2 * math.pi * 1000 * t)
    p = os.path.join(tmp_path, "a.wav")
    audio.write_wav(p, x, rate)
    y, r = audio.read_wav(p)
    assert r == rate and y.shape == (rate, 1) and (y[:, 0] - x).abs().max() < 1e-4
    fb = audio.mel_filterbank(40, 400, rate)
    assert fb.shape == (40, 201) and (fb >= 0).all() and (fb.sum(1) > 0).all()
    lm = audio.log_mel(x, rate)
    assert lm.shape == (101, 40)
    peak = lm.mean(0).argmax().item()
    centre = audio.mel_to_hz(audio.hz_to_mel(0) + (peak + 1) * (audio.hz_to_mel(8000) - audio.hz_to_mel(0)) / 41)
    assert 800 < centre < 1250
    d = audio.dct_matrix(13, 40)
    assert torch.allclose(d @ d.t(), torch.eye(13), atol=1e-5)
    assert audio.mfcc(x, rate).shape == (101, 13)
    nn.manual_seed(0)
    clf = audio.Classifier(4, width=4)
    assert tuple(clf(T.from_torch(lm[None, None])).shape) == (1, 4)


def test_envs_and_gae():
    env = rl.CartPole(seed=1)
    obs, total, done = env.reset(), 0, False
    while not done:
        obs, r, done = env.step(1)   # always push right: falls quickly
        total += r
    assert 5 <= total <= 15
    ch = rl.Chain(n=4, horizon=6)
    ch.reset()
    assert [ch.step(1)[1] for _ in range(5)] == [0.0, 0.0, 0.0, 1.0, 1.0]
    adv, ret = rl.gae([1.0, 1.0], [0.5, 0.5], [False, True], 9.0, gamma=0.5, lam=1.0)
    assert abs(adv[1] - 0.5) < 1e-9 and abs(adv[0] - (1 + 0.5 * 0.5 - 0.5 + 0.5 * 0.5)) < 1e-9 and ret[1] == 1.0


def test_dqn_learns_chain_and_ppo_improves_cartpole():
    env = rl.Chain(n=4, horizon=20)
    agent = rl.DQN(env.observations, env.actions, hidden=32, lr=5e-3, batch=32, target_every=50, eps=(1.0, 0.05, 600), seed=0)
    for _ in range(60):
        obs, done = env.reset(), False
        while not done:
            a = agent.act(obs)
            nxt, r, done = env.step(a)
            agent.observe(obs, a, r, nxt, done)
            obs = nxt
    obs, done, total = env.reset(), False, 0.0
    while not done:
        obs, r, done = env.step(agent.act(obs, greedy=True))
        total += r
    assert total >= 10, total      # the greedy policy walks to the end and stays there

    env = rl.CartPole(seed=0, max_steps=200)
    ppo = rl.PPO(4, 2, hidden=32, lr=3e-3, minibatch=128, epochs=4, seed=0)
    lengths = []
    for _ in range(12):
        O, A, L, R, V, D = [], [], [], [], [], []
        obs, ep = env.reset(), 0
        for _ in range(512):
            a, lp, v = ppo.act(obs)
            nxt, r, done = env.step(a)
            O.append(obs); A.append(a); L.append(lp); R.append(r); V.append(v); D.append(done)
            ep += 1
            obs = nxt
            if done:
                lengths.append(ep)
                obs, ep = env.reset(), 0
        ppo.update(O, A, L, R, V, D, ppo.act(obs)[2])
    assert sum(lengths[-5:]) / 5 > 1.5 * sum(lengths[:5]) / 5, (lengths[:5], lengths[-5:])
