"""Board games, negamax tree search on the true game model, AlphaZero self-play training on tic-tac-toe."""
import torch


def test_line_games_rules():
    from noeira_b200.envs import ConnectFour, TicTacToe
    g = TicTacToe()
    assert g.lines.shape == (8, 9) and g.n_actions == 9
    b = g.initial(2)
    b[0, [0, 1]] = 1.0                                             # mover has two in the top row
    b[0, [3, 4]] = -1.0
    nb, r, done = g.step(b, torch.tensor([2, 4]))
    assert r.tolist() == [1.0, 0.0] and done.tolist() == [True, False]
    assert torch.equal(nb[1], -torch.eye(9)[4]) and not g.legal(nb)[1, 4]
    c4 = ConnectFour()
    assert c4.lines.shape[0] == 69 and c4.n_actions == 7
    b = c4.initial(1)
    for _ in range(3):                                             # mover stacks column 2, opponent column 5
        b, r, d = c4.step(b, torch.tensor([2]))
        b, r, d = c4.step(b, torch.tensor([5]))
    grid = b.reshape(6, 7)
    assert grid[5, 2] == 1 and grid[3, 2] == 1 and grid[5, 5] == -1 and grid[2, 2] == 0     # stones fall to the bottom
    b, r, d = c4.step(b, torch.tensor([2]))
    assert r.item() == 1.0 and d.item()                            # four in a column
    full = c4.initial(1)
    full.reshape(6, 7)[:, 0] = torch.tensor([1., -1, 1, -1, 1, -1])
    assert not c4.legal(full)[0, 0] and c4.legal(full)[0, 1]


def test_search_on_the_true_model_wins_and_blocks():
    from noeira_b200.agents.alphazero import AlphaZeroAgent, AlphaZeroConfig
    from noeira_b200.envs import TicTacToe
    ag = AlphaZeroAgent(TicTacToe(), AlphaZeroConfig(hidden=16, n_simulations=120, seed=0))
    b = ag.game.initial(2)
    b[0, [0, 1]] = 1.0
    b[0, [3, 4]] = -1.0                                            # both sides threaten: taking the win comes first
    b[1, [3, 4]] = -1.0
    b[1, 0] = 1.0                                                  # the opponent threatens cell 5: block
    pi, v, a = ag.act(b)
    assert a.tolist() == [2, 5], (a, pi)
    assert v[0] > 0.3 and abs(float(pi.sum(1)[0]) - 1) < 1e-5
    assert (pi[~ag.game.legal(b)] == 0).all()                       # no visit ever enters an occupied cell


def test_loss_gradients_match_autograd():
    from noeira_b200.agents.alphazero import AlphaZeroAgent, AlphaZeroConfig
    from noeira_b200.envs import TicTacToe
    ag = AlphaZeroAgent(TicTacToe(), AlphaZeroConfig(hidden=8, value_coef=0.7))
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(6, 9, generator=g, requires_grad=True)
    vpre = torch.randn(6, generator=g, requires_grad=True)
    pi = torch.softmax(torch.randn(6, 9, generator=g), -1)
    z = torch.sign(torch.randn(6, generator=g))
    ref = -(pi * torch.log_softmax(logits, -1)).sum(-1).mean() + 0.7 * ((z - torch.tanh(vpre)) ** 2).mean()
    ref.backward()
    loss, dl, dv, _, _ = ag.loss_and_grads(logits.detach(), torch.tanh(vpre.detach()), pi, z)
    assert abs(float(loss) - float(ref.detach())) < 1e-6
    assert torch.allclose(dl, logits.grad, atol=1e-6) and torch.allclose(dv, vpre.grad, atol=1e-6)


def test_self_play_training_on_tictactoe():
    from noeira_b200.agents.alphazero import AlphaZeroAgent, AlphaZeroConfig
    from noeira_b200.envs import TicTacToe
    ag = AlphaZeroAgent(TicTacToe(), AlphaZeroConfig(hidden=64, n_simulations=30, batch=128, lr=3e-3, seed=0))
    losses = []
    for it in range(6):
        n = ag.self_play(48)
        assert n >= 48 * 5
        for _ in range(30):
            losses.append(ag.train_step()["loss"])
    z = ag.buf_z[: ag.size]
    assert set(z.unique().tolist()) <= {-1.0, 0.0, 1.0}
    assert sum(losses[-10:]) / 10 < sum(losses[:10]) / 10          # the network learns the search's targets
    w, d, l = ag.play_vs_random(64, agent_first=True)
    w2, d2, l2 = ag.play_vs_random(64, agent_first=False)
    assert l <= 1 and l2 <= 8 and w > 48 and w2 > 4 * l2, ((w, d, l), (w2, d2, l2))
    # the raw policy (no search) has picked up something too: it beats random more often than it loses
    w3, d3, l3 = ag.play_vs_random(64, agent_first=True, use_search=False)
    assert w3 > l3
