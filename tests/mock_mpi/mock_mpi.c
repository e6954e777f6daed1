/* A stand-in for an MPI library with the MPICH binary interface, enough of it for the MPI transport's tests
 * (there is no MPI installation in the image).  Point-to-point only: MPI_Isend copies the message into a queue
 * and completes at once, bytes travel over Unix stream sockets (one per ordered pair of ranks, opened by the
 * sender), MPI_Irecv / MPI_Iprobe match (communicator, source, tag) in arrival order per source, every call
 * makes progress.  Rank and size come from MOCK_MPI_RANK / MOCK_MPI_SIZE, else from CCL_LOCAL_RANK /
 * CCL_LOCAL_SIZE; with MOCK_MPI_REVERSE=1 the ranks are numbered the other way round (so that a caller cannot
 * assume that MPI ranks equal its own).  The sockets live in MOCK_MPI_DIR.
 *
 * Build: cc -shared -fPIC -O1 -o libmockmpi.so mock_mpi.c -lpthread */
#define _GNU_SOURCE
#include <errno.h>
#include <fcntl.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Request;
typedef struct {
    int count_lo;
    int count_hi_and_cancelled;
    int MPI_SOURCE;
    int MPI_TAG;
    int MPI_ERROR;
} MPI_Status;

#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_COMM_WORLD 0x44000000
#define MPI_REQUEST_NULL 0x2c000000
#define MPI_ANY_SOURCE (-2)
#define MPI_ANY_TAG (-1)
#define MPI_STATUS_IGNORE ((MPI_Status*)1)
#define MAX_RANKS 64

struct frame { /* on the wire, in front of the payload */
    int32_t comm;
    int32_t tag;
    uint64_t len;
};

struct msg { /* arrived, not yet received */
    struct msg* next;
    int comm, tag, src;
    uint64_t len;
    char* data;
};

struct outbuf { /* bytes still to be written to one peer */
    char* data;
    size_t len, off;
    struct outbuf* next;
};

struct rreq { /* a posted receive */
    int used, done, comm, src, tag;
    uint64_t seq; /* posting order: receives that could take the same message take them in this order */
    void* buf;
    uint64_t cap, got;
    int got_src, got_tag;
};

static pthread_mutex_t mu = PTHREAD_MUTEX_INITIALIZER;
static int g_init, g_fin, g_rank, g_size, g_listen = -1, g_next_comm = 1;
static char g_dir[80];
static int out_fd[MAX_RANKS], in_fd[MAX_RANKS];
static struct outbuf *out_head[MAX_RANKS], *out_tail[MAX_RANKS];
static struct msg *q_head[MAX_RANKS], *q_tail[MAX_RANKS];
/* partially read frame per source */
static struct frame in_hdr[MAX_RANKS];
static size_t in_hdr_got[MAX_RANKS];
static struct msg* in_cur[MAX_RANKS];
static uint64_t in_cur_got[MAX_RANKS];
#define MAX_REQ 4096
static struct rreq reqs[MAX_REQ];
static uint64_t g_post_seq;

static int env_int(const char* a, const char* b, int dflt) {
    const char* v = getenv(a);
    if (!v && b)
        v = getenv(b);
    return v ? atoi(v) : dflt;
}

static void set_nonblock(int fd) {
    fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK);
}

static void sock_path(struct sockaddr_un* a, int rank) {
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    snprintf(a->sun_path, sizeof(a->sun_path), "%s/mockmpi.%d", g_dir, rank);
}

static int connect_to(int peer) {
    struct sockaddr_un a;
    sock_path(&a, peer);
    for (int tries = 0; tries < 3000; tries++) {
        int fd = socket(AF_UNIX, SOCK_STREAM, 0);
        if (connect(fd, (struct sockaddr*)&a, sizeof(a)) == 0) {
            int32_t me = g_rank;
            if (write(fd, &me, sizeof(me)) != sizeof(me)) {
                close(fd);
                return -1;
            }
            set_nonblock(fd);
            return fd;
        }
        close(fd);
        struct timespec ts = { 0, 10 * 1000 * 1000 };
        nanosleep(&ts, NULL);
    }
    return -1;
}

static void try_match(struct rreq* r);

static void progress(void) {
    /* new connections: the first four bytes name the sender */
    for (;;) {
        int fd = accept(g_listen, NULL, NULL);
        if (fd < 0)
            break;
        int32_t who = -1;
        size_t got = 0;
        while (got < sizeof(who)) {
            ssize_t n = read(fd, (char*)&who + got, sizeof(who) - got);
            if (n > 0)
                got += (size_t)n;
            else if (n == 0 || (errno != EAGAIN && errno != EINTR))
                break;
        }
        if (who < 0 || who >= g_size) {
            close(fd);
            continue;
        }
        set_nonblock(fd);
        in_fd[who] = fd;
    }
    /* outgoing queues */
    for (int p = 0; p < g_size; p++) {
        while (out_head[p]) {
            struct outbuf* o = out_head[p];
            ssize_t n = write(out_fd[p], o->data + o->off, o->len - o->off);
            if (n <= 0)
                break;
            o->off += (size_t)n;
            if (o->off < o->len)
                break;
            out_head[p] = o->next;
            if (!out_head[p])
                out_tail[p] = NULL;
            free(o->data);
            free(o);
        }
    }
    /* incoming bytes */
    for (int s = 0; s < g_size; s++) {
        if (in_fd[s] < 0)
            continue;
        for (;;) {
            if (!in_cur[s]) {
                ssize_t n = read(in_fd[s], (char*)&in_hdr[s] + in_hdr_got[s], sizeof(struct frame) - in_hdr_got[s]);
                if (n <= 0)
                    break;
                in_hdr_got[s] += (size_t)n;
                if (in_hdr_got[s] < sizeof(struct frame))
                    break;
                struct msg* m = (struct msg*)calloc(1, sizeof(*m));
                m->comm = in_hdr[s].comm;
                m->tag = in_hdr[s].tag;
                m->src = s;
                m->len = in_hdr[s].len;
                m->data = (char*)malloc(m->len ? m->len : 1);
                in_cur[s] = m;
                in_cur_got[s] = 0;
                in_hdr_got[s] = 0;
            }
            struct msg* m = in_cur[s];
            if (in_cur_got[s] < m->len) {
                ssize_t n = read(in_fd[s], m->data + in_cur_got[s], m->len - in_cur_got[s]);
                if (n <= 0)
                    break;
                in_cur_got[s] += (uint64_t)n;
                if (in_cur_got[s] < m->len)
                    continue;
            }
            if (q_tail[s])
                q_tail[s]->next = m;
            else
                q_head[s] = m;
            q_tail[s] = m;
            in_cur[s] = NULL;
        }
    }
    /* posted receives, in posting order */
    uint64_t after = 0;
    for (;;) {
        int best = -1;
        for (int i = 0; i < MAX_REQ; i++)
            if (reqs[i].used && !reqs[i].done && reqs[i].seq > after && (best < 0 || reqs[i].seq < reqs[best].seq))
                best = i;
        if (best < 0)
            break;
        after = reqs[best].seq;
        try_match(&reqs[best]);
    }
}

static struct msg* find_msg(int comm, int src, int tag, int take) {
    int lo = src == MPI_ANY_SOURCE ? 0 : src, hi = src == MPI_ANY_SOURCE ? g_size - 1 : src;
    for (int s = lo; s <= hi; s++) {
        struct msg* prev = NULL;
        for (struct msg* m = q_head[s]; m; prev = m, m = m->next) {
            if (m->comm != comm || (tag != MPI_ANY_TAG && m->tag != tag))
                continue;
            if (take) {
                if (prev)
                    prev->next = m->next;
                else
                    q_head[s] = m->next;
                if (q_tail[s] == m)
                    q_tail[s] = prev;
                m->next = NULL;
            }
            return m;
        }
    }
    return NULL;
}

static void try_match(struct rreq* r) {
    struct msg* m = find_msg(r->comm, r->src, r->tag, 1);
    if (!m)
        return;
    uint64_t n = m->len < r->cap ? m->len : r->cap;
    if (n)
        memcpy(r->buf, m->data, n);
    r->got = n;
    r->got_src = m->src;
    r->got_tag = m->tag;
    r->done = 1;
    free(m->data);
    free(m);
}

static void fill_status(MPI_Status* st, int src, int tag, uint64_t n) {
    if (st == MPI_STATUS_IGNORE || !st)
        return;
    st->count_lo = (int)(n & 0x7fffffff);
    st->count_hi_and_cancelled = 0;
    st->MPI_SOURCE = src;
    st->MPI_TAG = tag;
    st->MPI_ERROR = MPI_SUCCESS;
}

int MPI_Init_thread(int* argc, char*** argv, int required, int* provided) {
    (void)argc;
    (void)argv;
    pthread_mutex_lock(&mu);
    if (!g_init) {
        g_size = env_int("MOCK_MPI_SIZE", "CCL_LOCAL_SIZE", 1);
        g_rank = env_int("MOCK_MPI_RANK", "CCL_LOCAL_RANK", 0);
        if (env_int("MOCK_MPI_REVERSE", NULL, 0))
            g_rank = g_size - 1 - g_rank;
        const char* d = getenv("MOCK_MPI_DIR");
        snprintf(g_dir, sizeof(g_dir), "%s", d ? d : "/tmp");
        for (int i = 0; i < MAX_RANKS; i++)
            out_fd[i] = in_fd[i] = -1;
        struct sockaddr_un a;
        sock_path(&a, g_rank);
        unlink(a.sun_path);
        g_listen = socket(AF_UNIX, SOCK_STREAM, 0);
        if (g_size > MAX_RANKS || bind(g_listen, (struct sockaddr*)&a, sizeof(a)) != 0 || listen(g_listen, MAX_RANKS) != 0) {
            pthread_mutex_unlock(&mu);
            return MPI_ERR_OTHER;
        }
        set_nonblock(g_listen);
        g_init = 1;
    }
    if (provided)
        *provided = env_int("MOCK_MPI_THREAD_LEVEL", NULL, required);
    pthread_mutex_unlock(&mu);
    return MPI_SUCCESS;
}

int MPI_Initialized(int* flag) {
    *flag = g_init;
    return MPI_SUCCESS;
}
int MPI_Finalized(int* flag) {
    *flag = g_fin;
    return MPI_SUCCESS;
}
int MPI_Query_thread(int* provided) {
    *provided = env_int("MOCK_MPI_THREAD_LEVEL", NULL, 3);
    return MPI_SUCCESS;
}

int MPI_Finalize(void) {
    pthread_mutex_lock(&mu);
    /* what was handed to MPI_Isend must still leave */
    for (int spin = 0; spin < 200000; spin++) {
        int pending = 0;
        progress();
        for (int p = 0; p < g_size; p++)
            pending |= out_head[p] != NULL;
        if (!pending)
            break;
        struct timespec ts = { 0, 50 * 1000 };
        nanosleep(&ts, NULL);
    }
    g_fin = 1;
    struct sockaddr_un a;
    sock_path(&a, g_rank);
    unlink(a.sun_path);
    pthread_mutex_unlock(&mu);
    return MPI_SUCCESS;
}

int MPI_Comm_rank(MPI_Comm c, int* r) {
    (void)c;
    *r = g_rank;
    return MPI_SUCCESS;
}
int MPI_Comm_size(MPI_Comm c, int* n) {
    (void)c;
    *n = g_size;
    return MPI_SUCCESS;
}
/* collective in a real MPI; here every rank counts its duplicates alike, which is all the matching needs */
int MPI_Comm_dup(MPI_Comm c, MPI_Comm* out) {
    (void)c;
    pthread_mutex_lock(&mu);
    *out = (int)(0x84000000u + (unsigned)g_next_comm++);
    pthread_mutex_unlock(&mu);
    return MPI_SUCCESS;
}
int MPI_Comm_free(MPI_Comm* c) {
    *c = 0;
    return MPI_SUCCESS;
}

int MPI_Get_library_version(char* v, int* len) {
    strcpy(v, "mock MPI (MPICH binary interface subset) for the transport tests");
    *len = (int)strlen(v);
    return MPI_SUCCESS;
}

int MPI_Isend(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request* req) {
    (void)dt;
    if (dest < 0 || dest >= g_size || count < 0)
        return MPI_ERR_OTHER;
    pthread_mutex_lock(&mu);
    if (out_fd[dest] < 0) {
        out_fd[dest] = connect_to(dest);
        if (out_fd[dest] < 0) {
            pthread_mutex_unlock(&mu);
            return MPI_ERR_OTHER;
        }
    }
    struct outbuf* o = (struct outbuf*)calloc(1, sizeof(*o));
    o->len = sizeof(struct frame) + (size_t)count;
    o->data = (char*)malloc(o->len);
    struct frame f = { comm, tag, (uint64_t)count };
    memcpy(o->data, &f, sizeof(f));
    if (count)
        memcpy(o->data + sizeof(f), buf, (size_t)count);
    if (out_tail[dest])
        out_tail[dest]->next = o;
    else
        out_head[dest] = o;
    out_tail[dest] = o;
    progress();
    *req = MPI_REQUEST_NULL; /* buffered: complete */
    pthread_mutex_unlock(&mu);
    return MPI_SUCCESS;
}

int MPI_Irecv(void* buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Request* req) {
    (void)dt;
    pthread_mutex_lock(&mu);
    int slot = -1;
    for (int i = 0; i < MAX_REQ; i++)
        if (!reqs[i].used) {
            slot = i;
            break;
        }
    if (slot < 0) {
        pthread_mutex_unlock(&mu);
        return MPI_ERR_OTHER;
    }
    struct rreq* r = &reqs[slot];
    memset(r, 0, sizeof(*r));
    r->used = 1;
    r->comm = comm;
    r->src = src;
    r->tag = tag;
    r->buf = buf;
    r->cap = (uint64_t)count;
    r->seq = ++g_post_seq;
    progress();
    *req = slot + 1; /* never equals MPI_REQUEST_NULL */
    pthread_mutex_unlock(&mu);
    return MPI_SUCCESS;
}

int MPI_Test(MPI_Request* req, int* flag, MPI_Status* st) {
    if (*req == MPI_REQUEST_NULL) {
        *flag = 1;
        fill_status(st, MPI_ANY_SOURCE, MPI_ANY_TAG, 0);
        return MPI_SUCCESS;
    }
    pthread_mutex_lock(&mu);
    progress();
    struct rreq* r = &reqs[*req - 1];
    *flag = r->done;
    if (r->done) {
        fill_status(st, r->got_src, r->got_tag, r->got);
        r->used = 0;
        *req = MPI_REQUEST_NULL;
    }
    pthread_mutex_unlock(&mu);
    return MPI_SUCCESS;
}

int MPI_Recv(void* buf, int count, MPI_Datatype dt, int src, int tag, MPI_Comm comm, MPI_Status* st) {
    MPI_Request r;
    int rc = MPI_Irecv(buf, count, dt, src, tag, comm, &r);
    if (rc != MPI_SUCCESS)
        return rc;
    for (;;) {
        int flag = 0;
        MPI_Test(&r, &flag, st);
        if (flag)
            return MPI_SUCCESS;
        struct timespec ts = { 0, 20 * 1000 };
        nanosleep(&ts, NULL);
    }
}

int MPI_Iprobe(int src, int tag, MPI_Comm comm, int* flag, MPI_Status* st) {
    pthread_mutex_lock(&mu);
    progress();
    struct msg* m = find_msg(comm, src, tag, 0);
    *flag = m != NULL;
    if (m)
        fill_status(st, m->src, m->tag, m->len);
    pthread_mutex_unlock(&mu);
    return MPI_SUCCESS;
}

int MPI_Get_count(const MPI_Status* st, MPI_Datatype dt, int* count) {
    (void)dt;
    *count = st->count_lo;
    return MPI_SUCCESS;
}
