"""Three small generative models on 2-D / image-shaped toy data (reference: examples/vae, examples/gan,
examples/diffusion).  Each ``*_main`` returns its loss history."""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def ring(n, gen):
    """Eight Gaussians on a circle."""
    k = torch.randint(0, 8, (n,), generator=gen)
    ang = k.float() * math.pi / 4
    return torch.stack([ang.cos(), ang.sin()], 1) * 2 + 0.05 * torch.randn(n, 2, generator=gen)


def vae_main(steps=200, log=print):
    import mimir_b200.tensor as T
    from mimir_b200 import distributions as D
    from mimir_b200 import nn, optim
    nn.manual_seed(0)
    gen = torch.Generator().manual_seed(0)
    enc = nn.Sequential(nn.Linear(2, 32), nn.Tanh(), nn.Linear(32, 4))      # mean and log-variance of a 2-D code
    dec = nn.Sequential(nn.Linear(2, 32), nn.Tanh(), nn.Linear(32, 2))
    opt = optim.Adam(enc.parameters() + dec.parameters(), lr=3e-3)
    prior = D.Normal(T.tensor([0.0, 0.0]), T.tensor([1.0, 1.0]))
    hist = []
    for s in range(steps):
        x = T.from_torch(ring(128, gen))
        h = enc(x)
        mu, logvar = h[:, :2], h[:, 2:]
        q = D.Normal(mu, T.exp(logvar * 0.5))
        z = q.rsample(seed=s)
        recon = T.mean(T.sum_((dec(z) - x) * (dec(z) - x), -1))
        kl = T.mean(T.sum_(D.kl(q, prior), -1))
        loss = recon + 0.05 * kl
        loss.backward()
        hist.append(float(loss.item()))
        opt.step()
        opt.zero_grad()
    log(f"vae: loss {hist[0]:.3f} -> {hist[-1]:.3f}")
    return hist


def gan_main(steps=150, log=print):
    import mimir_b200.tensor as T
    from mimir_b200 import nn, optim
    nn.manual_seed(0)
    gen = torch.Generator().manual_seed(0)
    G = nn.Sequential(nn.Linear(4, 32), nn.ReLU(), nn.Linear(32, 2))
    Dn = nn.Sequential(nn.Linear(2, 32), nn.LeakyReLU(0.2), nn.Linear(32, 1))
    og, od = optim.Adam(G.parameters(), lr=1e-3, betas=(0.5, 0.999)), optim.Adam(Dn.parameters(), lr=1e-3, betas=(0.5, 0.999))
    hist = []
    ones, zeros = T.from_torch(torch.ones(64, 1)), T.from_torch(torch.zeros(64, 1))
    for s in range(steps):
        real = T.from_torch(ring(64, gen))
        noise = T.from_torch(torch.randn(64, 4, generator=gen))
        fake = G(noise)
        T.realize(fake)
        d_loss = nn.loss.bce_with_logits(Dn(real), ones) + nn.loss.bce_with_logits(Dn(T.from_torch(fake.data().detach())), zeros)
        d_loss.backward()
        d_val = float(d_loss.item())
        od.step()
        od.zero_grad()
        g_loss = nn.loss.bce_with_logits(Dn(G(noise)), ones)      # non-saturating generator loss
        g_loss.backward()
        hist.append((d_val, float(g_loss.item())))
        og.step()
        og.zero_grad()
        od.zero_grad()
    log(f"gan: d {hist[-1][0]:.3f} g {hist[-1][1]:.3f}")
    return hist


def diffusion_main(steps=200, timesteps=50, log=print):
    import mimir_b200.tensor as T
    from mimir_b200 import nn, optim
    nn.manual_seed(0)
    gen = torch.Generator().manual_seed(0)
    betas = torch.linspace(1e-4, 0.2, timesteps)
    abar = torch.cumprod(1 - betas, 0)
    net = nn.Sequential(nn.Linear(3, 64), nn.SiLU(), nn.Linear(64, 64), nn.SiLU(), nn.Linear(64, 2))   # (x_t, t) -> noise
    opt = optim.Adam(net.parameters(), lr=2e-3)
    hist = []
    for _ in range(steps):
        x0 = ring(128, gen)
        t = torch.randint(0, timesteps, (128,), generator=gen)
        eps = torch.randn(128, 2, generator=gen)
        xt = abar[t].sqrt()[:, None] * x0 + (1 - abar[t]).sqrt()[:, None] * eps
        inp = T.from_torch(torch.cat([xt, (t.float() / timesteps)[:, None]], 1))
        loss = nn.loss.mse(net(inp), T.from_torch(eps))
        loss.backward()
        hist.append(float(loss.item()))
        opt.step()
        opt.zero_grad()
    # ancestral sampling
    with torch.no_grad():
        x = torch.randn(256, 2, generator=gen)
        for i in reversed(range(timesteps)):
            tt = torch.full((256, 1), i / timesteps)
            e = net(T.from_torch(torch.cat([x, tt], 1))).data()
            x = (x - betas[i] / (1 - abar[i]).sqrt() * e) / (1 - betas[i]).sqrt()
            if i:
                x = x + betas[i].sqrt() * torch.randn(256, 2, generator=gen)
    log(f"diffusion: loss {hist[0]:.3f} -> {hist[-1]:.3f}; sample radius {x.norm(dim=1).mean():.2f} (data: 2.0)")
    return hist, x


if __name__ == "__main__":
    vae_main()
    gan_main()
    diffusion_main()
